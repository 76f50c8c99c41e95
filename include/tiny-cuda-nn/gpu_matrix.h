/* tiny-cuda-nn/gpu_matrix.h of the B200-native stand-in: MatrixView<T> (what kernels index), GPUMatrixDynamic<T> (layout
 * chosen at run time) and GPUMatrix<T, layout>.  A matrix is m rows (features) by n columns (batch elements); column-major
 * ("AoS") keeps one batch element contiguous, row-major ("SoA") keeps one feature contiguous.  Call sites followed:
 * include/neural-graphics-primitives/nerf_network.h:94-124, :137-147, :332-340, common_operation.cuh:166-185,
 * src/testbed_nerf.cu:3771-3777. */
#pragma once
#include <tiny-cuda-nn/common.h>
#include <tiny-cuda-nn/gpu_memory.h>

TCNN_NAMESPACE_BEGIN

template <typename T>
struct MatrixView {
	TCNN_HOST_DEVICE MatrixView() : data{nullptr}, stride_i{0}, stride_j{0} {}
	TCNN_HOST_DEVICE MatrixView(T* data, uint32_t stride_i, uint32_t stride_j) : data{data}, stride_i{stride_i}, stride_j{stride_j} {}
	TCNN_HOST_DEVICE MatrixView(const MatrixView<std::remove_const_t<T>>& other) : data{other.data}, stride_i{other.stride_i}, stride_j{other.stride_j} {}
	TCNN_HOST_DEVICE T& operator()(uint32_t i, uint32_t j = 0) const { return data[(size_t)i * stride_i + (size_t)j * stride_j]; }
	TCNN_HOST_DEVICE void advance(uint32_t m, uint32_t n) { data += (size_t)m * stride_i + (size_t)n * stride_j; }
	TCNN_HOST_DEVICE void advance_rows(uint32_t m) { advance(m, 0); }
	TCNN_HOST_DEVICE void advance_cols(uint32_t n) { advance(0, n); }
	TCNN_HOST_DEVICE explicit operator bool() const { return data; }
	T* data;
	uint32_t stride_i, stride_j;
};

template <typename T>
class GPUMatrixDynamic;
template <typename T, MatrixLayout _layout = MatrixLayout::ColumnMajor>
class GPUMatrix;

class GPUMatrixBase {
public:
	virtual ~GPUMatrixBase() {}
	virtual size_t n_bytes() const = 0;
	virtual void set_data_unsafe(void* data) = 0;

	/* one workspace for several matrices, cut at 256-byte boundaries */
	static void allocate_shared_memory(GPUMemory<char>& memory, const std::vector<GPUMatrixBase*>& matrices) {
		size_t total = 0;
		for (auto* m : matrices) total += next_multiple(m->n_bytes(), (size_t)256);
		if (memory.bytes() < total) memory.resize(total);
		size_t offset = 0;
		for (auto* m : matrices) {
			m->set_data_unsafe(memory.data() + offset);
			offset += next_multiple(m->n_bytes(), (size_t)256);
		}
	}
	static GPUMemoryArena::Allocation allocate_shared_memory(cudaStream_t stream, const std::vector<GPUMatrixBase*>& matrices) {
		size_t total = 0;
		for (auto* m : matrices) total += next_multiple(m->n_bytes(), (size_t)256);
		auto alloc = allocate_workspace(stream, total);
		size_t offset = 0;
		for (auto* m : matrices) {
			m->set_data_unsafe(alloc.data() + offset);
			offset += next_multiple(m->n_bytes(), (size_t)256);
		}
		return alloc;
	}
};

template <typename T>
class GPUMatrixDynamic : public GPUMatrixBase {
public:
	using Type = T;

	/* owning, from the stream-ordered workspace */
	GPUMatrixDynamic(uint32_t m, uint32_t n, cudaStream_t stream, MatrixLayout layout = CM)
	    : m_rows{m}, m_cols{n}, m_layout{layout}, m_arena{std::make_shared<GPUMemoryArena::Allocation>(allocate_workspace(stream, (size_t)m * n * sizeof(T)))} {
		m_data = (T*)m_arena->data();
		set_stride_contiguous();
		/* defined contents: callers leave padding rows unwritten and feed the matrix to a network all the same
		 * (include/neural-graphics-primitives/nerf_network.h:137-139, :193-199), where stale NaN bits would spread */
		if (n_bytes()) CUDA_CHECK_THROW(cudaMemsetAsync(m_data, 0, n_bytes(), stream));
	}
	/* owning, plain device allocation */
	GPUMatrixDynamic(uint32_t m, uint32_t n, MatrixLayout layout = CM)
	    : m_rows{m}, m_cols{n}, m_layout{layout}, m_owned{std::make_shared<GPUMemory<uint8_t>>((size_t)m * n * sizeof(T))} {
		m_data = (T*)m_owned->data();
		set_stride_contiguous();
	}
	/* a view of memory someone else owns */
	GPUMatrixDynamic(T* data, uint32_t m, uint32_t n, MatrixLayout layout = CM, uint32_t stride = 0, std::shared_ptr<GPUMemory<uint8_t>> owned = nullptr,
	                 std::shared_ptr<GPUMemoryArena::Allocation> arena = nullptr)
	    : m_data{data}, m_rows{m}, m_cols{n}, m_layout{layout}, m_owned{owned}, m_arena{arena} {
		if (stride)
			m_stride = stride;
		else
			set_stride_contiguous();
	}
	GPUMatrixDynamic() : GPUMatrixDynamic{nullptr, 0, 0} {}
	GPUMatrixDynamic(const GPUMatrixDynamic<T>&) = default;
	GPUMatrixDynamic<T>& operator=(const GPUMatrixDynamic<T>&) = default;
	GPUMatrixDynamic(GPUMatrixDynamic<T>&&) = default;
	GPUMatrixDynamic<T>& operator=(GPUMatrixDynamic<T>&&) = default;
	virtual ~GPUMatrixDynamic() {}

	void set_data_unsafe(void* data) override { m_data = (T*)data; }
	void set_size_unsafe(uint32_t rows, uint32_t cols, uint32_t stride = 0) {
		m_rows = rows;
		m_cols = cols;
		if (stride)
			m_stride = stride;
		else
			set_stride_contiguous();
	}
	void set(T* data, uint32_t rows, uint32_t cols) {
		set_data_unsafe(data);
		set_size_unsafe(rows, cols);
	}
	void resize(uint32_t rows, uint32_t cols) {
		if (m_arena || m_owned) {
			m_arena.reset();
			m_owned = std::make_shared<GPUMemory<uint8_t>>((size_t)rows * cols * sizeof(T));
			m_data = (T*)m_owned->data();
		}
		set_size_unsafe(rows, cols);
	}

	uint32_t stride_contiguous() const { return m_layout == CM ? m_rows : m_cols; }
	bool is_contiguous() const { return m_stride == stride_contiguous(); }
	void set_stride_contiguous() { m_stride = stride_contiguous(); }

	GPUMatrixDynamic<T> slice(uint32_t offset_rows, uint32_t new_rows, uint32_t offset_cols, uint32_t new_cols) const {
		return GPUMatrixDynamic<T>{m_data + (m_layout == CM ? (offset_rows + (size_t)offset_cols * m_stride) : (offset_cols + (size_t)offset_rows * m_stride)),
		                           new_rows, new_cols, m_layout, m_stride, m_owned, m_arena};
	}
	GPUMatrixDynamic<T> slice_rows(uint32_t offset, uint32_t size) const { return slice(offset, size, 0, cols()); }
	GPUMatrixDynamic<T> slice_cols(uint32_t offset, uint32_t size) const { return slice(0, rows(), offset, size); }
	GPUMatrixDynamic<T> alias() const { return slice(0, rows(), 0, cols()); }

	MatrixView<T> view() const { return {data(), m_layout == CM ? 1u : m_stride, m_layout == CM ? m_stride : 1u}; }

	uint32_t rows() const { return m_rows; }
	uint32_t fan_out() const { return m_rows; }
	uint32_t m() const { return m_rows; }
	uint32_t cols() const { return m_cols; }
	uint32_t fan_in() const { return m_cols; }
	uint32_t n() const { return m_cols; }
	uint32_t stride() const { return m_stride; }
	uint32_t n_elements() const { return m_rows * m_cols; }
	size_t n_bytes() const override { return (size_t)m_rows * m_cols * sizeof(T); }
	T* data() const { return m_data; }
	MatrixLayout layout() const { return m_layout; }
	void set_layout(MatrixLayout layout) {
		m_layout = layout;
		set_stride_contiguous();
	}
	MatrixLayout transposed_layout() const { return m_layout == RM ? CM : RM; }

	GPUMatrixDynamic<T> transposed() const { return GPUMatrixDynamic<T>(m_data, m_cols, m_rows, transposed_layout(), m_stride, m_owned, m_arena); }
	GPUMatrix<T, RM> rm() const;
	GPUMatrix<T, CM> cm() const;

	void memset(int value) {
		if (!is_contiguous()) throw std::runtime_error("GPUMatrix::memset: the matrix is a strided slice");
		CUDA_CHECK_THROW(cudaMemset(data(), value, n_bytes()));
	}
	void memset_async(cudaStream_t stream, int value) {
		if (!is_contiguous()) throw std::runtime_error("GPUMatrix::memset_async: the matrix is a strided slice");
		CUDA_CHECK_THROW(cudaMemsetAsync(data(), value, n_bytes(), stream));
	}
	/* value in every entry; goes through the host, for set-up code only */
	void initialize_constant(float val) {
		std::vector<T> host((size_t)m_rows * m_cols, (T)val);
		CUDA_CHECK_THROW(cudaMemcpy(data(), host.data(), n_bytes(), cudaMemcpyHostToDevice));
	}
	std::vector<T> to_cpu_vector() const {
		std::vector<T> v((size_t)m_rows * m_cols);
		CUDA_CHECK_THROW(cudaMemcpy(v.data(), data(), n_bytes(), cudaMemcpyDeviceToHost));
		return v;
	}

protected:
	T* m_data = nullptr;
	uint32_t m_rows = 0, m_cols = 0, m_stride = 0;
	MatrixLayout m_layout = CM;
	std::shared_ptr<GPUMemory<uint8_t>> m_owned;
	std::shared_ptr<GPUMemoryArena::Allocation> m_arena;
};

template <typename T, MatrixLayout _layout>
class GPUMatrix : public GPUMatrixDynamic<T> {
public:
	static const MatrixLayout static_layout = _layout;
	static const MatrixLayout static_transposed_layout = _layout == RM ? CM : RM;

	GPUMatrix(uint32_t m, uint32_t n, cudaStream_t stream) : GPUMatrixDynamic<T>{m, n, stream, static_layout} {}
	GPUMatrix(uint32_t m, uint32_t n) : GPUMatrixDynamic<T>{m, n, static_layout} {}
	GPUMatrix(T* data, uint32_t m, uint32_t n, uint32_t stride = 0, std::shared_ptr<GPUMemory<uint8_t>> owned = nullptr,
	          std::shared_ptr<GPUMemoryArena::Allocation> arena = nullptr)
	    : GPUMatrixDynamic<T>{data, m, n, static_layout, stride, owned, arena} {}
	GPUMatrix() : GPUMatrix{nullptr, 0, 0} {}
	GPUMatrix(const GPUMatrixDynamic<T>& other) : GPUMatrixDynamic<T>{other} {
		if (other.layout() != static_layout) throw std::runtime_error("GPUMatrix: the dynamic matrix has the other layout");
	}
	GPUMatrix(GPUMatrixDynamic<T>&& other) : GPUMatrixDynamic<T>{std::move(other)} {
		if (this->layout() != static_layout) throw std::runtime_error("GPUMatrix: the dynamic matrix has the other layout");
	}
	GPUMatrix(const GPUMatrix<T, _layout>&) = default;
	GPUMatrix<T, _layout>& operator=(const GPUMatrix<T, _layout>&) = default;
	GPUMatrix(GPUMatrix<T, _layout>&&) = default;
	GPUMatrix<T, _layout>& operator=(GPUMatrix<T, _layout>&&) = default;
	virtual ~GPUMatrix() {}

	GPUMatrix<T, static_layout> slice(uint32_t offset_rows, uint32_t new_rows, uint32_t offset_cols, uint32_t new_cols) const {
		return ((GPUMatrixDynamic<T>*)this)->slice(offset_rows, new_rows, offset_cols, new_cols);
	}
	GPUMatrix<T, static_layout> slice_rows(uint32_t offset, uint32_t size) const { return ((GPUMatrixDynamic<T>*)this)->slice_rows(offset, size); }
	GPUMatrix<T, static_layout> slice_cols(uint32_t offset, uint32_t size) const { return ((GPUMatrixDynamic<T>*)this)->slice_cols(offset, size); }
	GPUMatrix<T, static_layout> alias() const { return ((GPUMatrixDynamic<T>*)this)->alias(); }
	GPUMatrix<T, static_transposed_layout> transposed() const {
		return GPUMatrix<T, static_transposed_layout>(this->m_data, this->m_cols, this->m_rows, this->m_stride, this->m_owned, this->m_arena);
	}
};

template <typename T>
GPUMatrix<T, RM> GPUMatrixDynamic<T>::rm() const {
	if (m_layout != RM) throw std::runtime_error("GPUMatrixDynamic::rm: the matrix is column-major");
	return GPUMatrix<T, RM>{m_data, m_rows, m_cols, m_stride, m_owned, m_arena};
}
template <typename T>
GPUMatrix<T, CM> GPUMatrixDynamic<T>::cm() const {
	if (m_layout != CM) throw std::runtime_error("GPUMatrixDynamic::cm: the matrix is row-major");
	return GPUMatrix<T, CM>{m_data, m_rows, m_cols, m_stride, m_owned, m_arena};
}

#if defined(__CUDACC__)
template <typename TOut, typename TIn>
__global__ void copy_view_kernel(const uint32_t n_elements, const uint32_t rows, MatrixView<const TIn> in, MatrixView<TOut> out) {
	const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
	if (i >= n_elements) return;
	const uint32_t col = i / rows, row = i - col * rows;
	out(row, col) = (TOut)in(row, col);
}

/* A dense column-major stand-in for a matrix of any layout or stride: the kernels behind the C interface read and write
 * one batch element as one contiguous row of `rows` values.  If the matrix already has that shape it is used in place;
 * otherwise a workspace copy is made (gather) or written back (scatter).  The copies are the price of a strided or
 * row-major operand on the layered path; the fused entry points never pay it. */
template <typename T>
class DenseColumns {
public:
	/* strided_ok: the consumer takes a column stride, so a column-major slice of a wider record is used in place too */
	DenseColumns(cudaStream_t stream, const GPUMatrixDynamic<T>& m, bool gather, bool strided_ok = false) : m_stream{stream}, m_matrix{m} {
		if (m.layout() == CM && (strided_ok || m.is_contiguous())) {
			m_data = m.data();
			return;
		}
		m_tmp = allocate_workspace(stream, std::max(m.n_bytes(), (size_t)16));
		m_data = (T*)m_tmp.data();
		m_copied = true;
		if (gather && m.n_elements())
			copy_view_kernel<T, T><<<n_blocks_linear(m.n_elements()), n_threads_linear, 0, stream>>>(m.n_elements(), m.m(), MatrixView<const T>(m.view()),
			                                                                                      MatrixView<T>{m_data, 1u, m.m()});
	}
	void scatter() {
		if (!m_copied || !m_matrix.n_elements()) return;
		copy_view_kernel<T, T><<<n_blocks_linear(m_matrix.n_elements()), n_threads_linear, 0, m_stream>>>(
		    m_matrix.n_elements(), m_matrix.m(), MatrixView<const T>{m_data, 1u, m_matrix.m()}, m_matrix.view());
	}
	T* data() const { return m_data; }
	bool copied() const { return m_copied; }

private:
	cudaStream_t m_stream;
	GPUMatrixDynamic<T> m_matrix;
	GPUMemoryArena::Allocation m_tmp;
	T* m_data = nullptr;
	bool m_copied = false;
};
#endif

TCNN_NAMESPACE_END
