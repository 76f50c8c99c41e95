/* <json/json.hpp> as the reference includes it (include/neural-graphics-primitives/testbed.h:23, nerf_network.h:23): tiny-cuda-nn
 * carries a copy of the single-header nlohmann/json library under this name.  That library is third-party code and is not
 * vendored here: this file forwards to the copy the build environment provides -- put a directory that holds
 * nlohmann/json.hpp on the include path (CMake: the nlohmann_json package's include directory). */
#pragma once
#if __has_include(<nlohmann/json.hpp>)
#include <nlohmann/json.hpp>
#else
#error "json/json.hpp: add the directory that contains nlohmann/json.hpp to the include path"
#endif

/* Fixed-size Eigen matrices.  The reference converts them through overloads on Eigen::MatrixBase<Derived>
 * (include/neural-graphics-primitives/json_binding.h:27-55).  Newer releases of the json library regard an Eigen vector as
 * an array-like container and prefer their own generic conversion, which needs insert() and does not compile.  These
 * overloads, found through the Eigen argument and more specialised than the generic one, restore the reference's reading:
 * a vector is a flat array, a matrix an array of rows. */
namespace Eigen {
template <typename Scalar, int Rows, int Cols, int Options, int MaxRows, int MaxCols>
class Matrix;

template <typename Scalar, int Rows, int Cols, int Options, int MaxRows, int MaxCols>
void from_json(const nlohmann::json& j, Matrix<Scalar, Rows, Cols, Options, MaxRows, MaxCols>& mat) {
	for (std::size_t row = 0; row < j.size(); ++row) {
		const auto& entry = j.at(row);
		if (entry.is_array()) {
			for (std::size_t col = 0; col < entry.size(); ++col) mat(row, col) = entry.at(col).template get<Scalar>();
		} else {
			mat(row) = entry.template get<Scalar>();
		}
	}
}
template <typename Scalar, int Rows, int Cols, int Options, int MaxRows, int MaxCols>
void to_json(nlohmann::json& j, const Matrix<Scalar, Rows, Cols, Options, MaxRows, MaxCols>& mat) {
	j = nlohmann::json::array();
	for (int row = 0; row < mat.rows(); ++row) {
		if (mat.cols() == 1) {
			j.push_back(mat(row));
		} else {
			nlohmann::json values = nlohmann::json::array();
			for (int col = 0; col < mat.cols(); ++col) values.push_back(mat(row, col));
			j.push_back(values);
		}
	}
}
}  // namespace Eigen
