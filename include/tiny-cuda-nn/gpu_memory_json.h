/* tiny-cuda-nn/gpu_memory_json.h of the B200-native stand-in: device arrays to and from json binary blobs, which is how
 * the reference's snapshots carry parameters, the density grid and the accumulated motion
 * (include/neural-graphics-primitives/nerf_network.h:1192-1235, src/testbed.cu:3130-3260). */
#pragma once
#include <tiny-cuda-nn/common.h>
#include <tiny-cuda-nn/gpu_memory.h>

#include <json/json.hpp>

TCNN_NAMESPACE_BEGIN
using json = nlohmann::json;

inline json::binary_t gpu_memory_to_json_binary(const void* gpu_data, size_t n_bytes) {
	json::binary_t data_cpu;
	data_cpu.resize(n_bytes);
	if (n_bytes) CUDA_CHECK_THROW(cudaMemcpy(data_cpu.data(), gpu_data, n_bytes, cudaMemcpyDeviceToHost));
	return data_cpu;
}
inline void json_binary_to_gpu_memory(const json::binary_t& cpu_data, void* gpu_data, size_t n_bytes) {
	if (cpu_data.size() != n_bytes) throw std::runtime_error("json_binary_to_gpu_memory: the blob holds " + std::to_string(cpu_data.size()) + " bytes, the array " + std::to_string(n_bytes));
	if (n_bytes) CUDA_CHECK_THROW(cudaMemcpy(gpu_data, cpu_data.data(), n_bytes, cudaMemcpyHostToDevice));
}

template <typename T>
inline void to_json(json& j, const GPUMemory<T>& gpu_data) {
	j = gpu_memory_to_json_binary(gpu_data.data(), gpu_data.get_bytes());
}
template <typename T>
inline void from_json(const json& j, GPUMemory<T>& gpu_data) {
	if (j.is_binary()) {
		const json::binary_t& cpu_data = j.get_binary();
		gpu_data.resize(cpu_data.size() / sizeof(T));
		json_binary_to_gpu_memory(cpu_data, gpu_data.data(), gpu_data.get_bytes());
	} else if (j.is_object()) {
		/* some msgpack writers wrap the payload: {"bytes": ..., "subtype": ...} */
		const json::binary_t& cpu_data = j.at("bytes").get_binary();
		gpu_data.resize(cpu_data.size() / sizeof(T));
		json_binary_to_gpu_memory(cpu_data, gpu_data.data(), gpu_data.get_bytes());
	} else {
		throw std::runtime_error("from_json(GPUMemory): the entry is not a binary blob");
	}
}

TCNN_NAMESPACE_END
