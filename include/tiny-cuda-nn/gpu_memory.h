/* tiny-cuda-nn/gpu_memory.h of the B200-native stand-in: GPUMemory<T> (an owning device array), the stream-ordered
 * workspace arena (GPUMemoryArena::Allocation, allocate_workspace, allocate_workspace_and_distribute) and the byte
 * accounting the reference prints (src/testbed.cu:381).  Call sites followed: src/testbed_nerf.cu:2606, :3217, :3723-3749,
 * src/marching_cubes.cu:801, include/neural-graphics-primitives/nerf_network.h:1003-1012.
 *
 * The arena is CUDA's stream-ordered allocator: every workspace is a cudaMallocAsync block of the device's default memory
 * pool, whose release threshold is raised once so that freed blocks stay in the pool -- after the first training step no
 * allocation reaches the driver, and a block freed on a stream is reused by the next request on that stream without a
 * synchronisation.  A workspace belongs to its stream: it must be released before the stream is destroyed. */
#pragma once
#include <tiny-cuda-nn/common.h>

#include <atomic>
#include <cstring>
#include <tuple>
#include <unordered_map>

TCNN_NAMESPACE_BEGIN

namespace detail {
inline std::atomic<size_t>& bytes_allocated_counter() {
	static std::atomic<size_t> s_total{0};
	return s_total;
}
}  // namespace detail
inline size_t total_n_bytes_allocated() { return detail::bytes_allocated_counter().load(); }

template <typename T>
class GPUMemory {
public:
	GPUMemory() = default;
	GPUMemory(size_t size, bool managed = false) : m_managed{managed} { resize(size); }
	GPUMemory(const GPUMemory<T>& other) : m_managed{other.m_managed} { copy_from_device(other); }
	GPUMemory<T>& operator=(GPUMemory<T>&& other) {
		std::swap(m_data, other.m_data);
		std::swap(m_size, other.m_size);
		std::swap(m_managed, other.m_managed);
		return *this;
	}
	GPUMemory(GPUMemory<T>&& other) { *this = std::move(other); }
	GPUMemory<T>& operator=(const GPUMemory<T>& other) {
		m_managed = other.m_managed;
		copy_from_device(other);
		return *this;
	}
	~GPUMemory() {
		try {
			free_memory();
		} catch (const std::exception& e) {
			if (std::string{e.what()}.find("driver shutting down") == std::string::npos) std::cerr << "Could not free memory: " << e.what() << std::endl;
		}
	}

	void allocate_memory(size_t n_bytes) {
		if (n_bytes == 0) return;
		void* p = nullptr;
		if (m_managed)
			CUDA_CHECK_THROW(cudaMallocManaged(&p, n_bytes));
		else
			CUDA_CHECK_THROW(cudaMalloc(&p, n_bytes));
		m_data = (T*)p;
		detail::bytes_allocated_counter() += n_bytes;
	}
	void free_memory() {
		if (!m_data) return;
		CUDA_CHECK_THROW(cudaFree(m_data));
		detail::bytes_allocated_counter() -= get_bytes();
		m_data = nullptr;
		m_size = 0;
	}
	/* contents are not kept */
	void resize(size_t size) {
		if (m_size == size) return;
		free_memory();
		m_size = size;
		try {
			allocate_memory(size * sizeof(T));
		} catch (...) {
			m_size = 0;
			throw;
		}
	}
	void enlarge(size_t size) {
		if (size > m_size) resize(size);
	}
	void memset(int value, size_t num_elements, size_t offset = 0) {
		if (num_elements + offset > m_size) throw std::runtime_error("GPUMemory::memset: out of bounds");
		CUDA_CHECK_THROW(cudaMemset(m_data + offset, value, num_elements * sizeof(T)));
	}
	void memset(int value) { memset(value, m_size); }
	void memset_async(cudaStream_t stream, int value) {
		if (m_size) CUDA_CHECK_THROW(cudaMemsetAsync(m_data, value, get_bytes(), stream));
	}

	void copy_from_host(const T* host_data, size_t num_elements) {
		if (num_elements > m_size) throw std::runtime_error("GPUMemory::copy_from_host: more elements than the array holds");
		if (num_elements) CUDA_CHECK_THROW(cudaMemcpy(m_data, host_data, num_elements * sizeof(T), cudaMemcpyHostToDevice));
	}
	void copy_from_host(const std::vector<T>& data, size_t num_elements) {
		if (data.size() < num_elements) throw std::runtime_error("GPUMemory::copy_from_host: the vector is shorter than the request");
		copy_from_host(data.data(), num_elements);
	}
	void copy_from_host(const T* data) { copy_from_host(data, m_size); }
	void copy_from_host(const std::vector<T>& data) {
		if (data.size() < m_size) throw std::runtime_error("GPUMemory::copy_from_host: the vector is shorter than the array");
		copy_from_host(data.data(), m_size);
	}
	void enlarge_and_copy_from_host(const T* data, size_t num_elements) {
		enlarge(num_elements);
		copy_from_host(data, num_elements);
	}
	void enlarge_and_copy_from_host(const std::vector<T>& data) { enlarge_and_copy_from_host(data.data(), data.size()); }
	void resize_and_copy_from_host(const T* data, size_t num_elements) {
		resize(num_elements);
		copy_from_host(data, num_elements);
	}
	void resize_and_copy_from_host(const std::vector<T>& data) { resize_and_copy_from_host(data.data(), data.size()); }

	void copy_to_host(T* host_data, size_t num_elements) const {
		if (num_elements > m_size) throw std::runtime_error("GPUMemory::copy_to_host: more elements than the array holds");
		if (num_elements) CUDA_CHECK_THROW(cudaMemcpy(host_data, m_data, num_elements * sizeof(T), cudaMemcpyDeviceToHost));
	}
	void copy_to_host(std::vector<T>& data, size_t num_elements) const {
		if (data.size() < num_elements) throw std::runtime_error("GPUMemory::copy_to_host: the vector is shorter than the request");
		copy_to_host(data.data(), num_elements);
	}
	void copy_to_host(T* data) const { copy_to_host(data, m_size); }
	void copy_to_host(std::vector<T>& data) const {
		if (data.size() < m_size) throw std::runtime_error("GPUMemory::copy_to_host: the vector is shorter than the array");
		copy_to_host(data.data(), m_size);
	}
	void copy_from_device(const GPUMemory<T>& other, size_t size) {
		if (size == 0) return;
		if (m_size < size) resize(size);
		CUDA_CHECK_THROW(cudaMemcpy(m_data, other.m_data, size * sizeof(T), cudaMemcpyDeviceToDevice));
	}
	void copy_from_device(const GPUMemory<T>& other) { copy_from_device(other, other.m_size); }
	GPUMemory<T> copy(size_t size) const {
		GPUMemory<T> result{size};
		result.copy_from_device(*this, size);
		return result;
	}
	GPUMemory<T> copy() const { return copy(m_size); }

	T* data() const { return m_data; }
	TCNN_HOST_DEVICE T& operator[](size_t idx) const { return m_data[idx]; }
	TCNN_HOST_DEVICE T& operator[](uint32_t idx) const { return m_data[idx]; }
	size_t get_num_elements() const { return m_size; }
	size_t size() const { return get_num_elements(); }
	size_t get_bytes() const { return m_size * sizeof(T); }
	size_t bytes() const { return get_bytes(); }

private:
	T* m_data = nullptr;
	size_t m_size = 0;
	bool m_managed = false;
};

/* ---- stream-ordered workspace */
namespace detail {
inline void keep_pool_memory(int device) {
	static std::unordered_map<int, bool> s_done;
	if (s_done[device]) return;
	cudaMemPool_t pool;
	CUDA_CHECK_THROW(cudaDeviceGetDefaultMemPool(&pool, device));
	uint64_t threshold = UINT64_MAX;
	CUDA_CHECK_THROW(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
	s_done[device] = true;
}
}  // namespace detail

class GPUMemoryArena {
public:
	class Allocation {
	public:
		Allocation() = default;
		Allocation(cudaStream_t stream, size_t n_bytes) : m_stream{stream}, m_bytes{n_bytes} {
			if (!n_bytes) return;
			int device = 0;
			CUDA_CHECK_THROW(cudaGetDevice(&device));
			detail::keep_pool_memory(device);
			CUDA_CHECK_THROW(cudaMallocAsync((void**)&m_data, n_bytes, stream));
			detail::bytes_allocated_counter() += n_bytes;
		}
		~Allocation() { release(); }
		Allocation(const Allocation&) = delete;
		Allocation& operator=(const Allocation&) = delete;
		Allocation& operator=(Allocation&& other) {
			std::swap(m_stream, other.m_stream);
			std::swap(m_data, other.m_data);
			std::swap(m_bytes, other.m_bytes);
			return *this;
		}
		Allocation(Allocation&& other) { *this = std::move(other); }
		uint8_t* data() { return m_data; }
		const uint8_t* data() const { return m_data; }
		cudaStream_t stream() const { return m_stream; }
		size_t size() const { return m_bytes; }

	private:
		void release() {
			if (!m_data) return;
			cudaFreeAsync(m_data, m_stream);
			detail::bytes_allocated_counter() -= m_bytes;
			m_data = nullptr;
			m_bytes = 0;
		}
		cudaStream_t m_stream = nullptr;
		uint8_t* m_data = nullptr;
		size_t m_bytes = 0;
	};
};

inline GPUMemoryArena::Allocation allocate_workspace(cudaStream_t stream, size_t n_bytes) {
	/* an empty request still yields a valid pointer, as callers pass it on unconditionally */
	return GPUMemoryArena::Allocation{stream, n_bytes ? n_bytes : 1};
}

/* gives the pool's cached blocks of the current device back to the driver */
inline void free_gpu_memory_arena(cudaStream_t stream) {
	(void)stream;
	int device = 0;
	if (cudaGetDevice(&device) != cudaSuccess) return;
	cudaMemPool_t pool;
	if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) cudaMemPoolTrimTo(pool, 0);
}
inline void free_all_gpu_memory_arenas() { free_gpu_memory_arena(nullptr); }

namespace detail {
static constexpr size_t workspace_alignment = 256; /* every sub-array starts on a 256-byte boundary */
inline size_t align_to_workspace(size_t bytes) { return next_multiple(bytes, workspace_alignment); }

template <typename First, typename... Rest>
struct Distribute {
	template <typename... Sizes>
	static std::tuple<First*, Rest*...> run(uint8_t* base, size_t first_size, Sizes... sizes) {
		auto head = std::make_tuple((First*)base);
		if constexpr (sizeof...(Rest) == 0)
			return head;
		else
			return std::tuple_cat(head, Distribute<Rest...>::run(base + align_to_workspace(first_size * sizeof(First)), sizes...));
	}
};
template <typename... Types, size_t... I>
size_t workspace_bytes(std::index_sequence<I...>, const size_t* sizes) {
	size_t total = 0;
	size_t each[] = {align_to_workspace(sizes[I] * sizeof(Types))...};
	for (size_t b : each) total += b;
	return total;
}
}  // namespace detail

/* one workspace cut into typed arrays: sizes are element counts, one per type (src/testbed_nerf.cu:3723-3749) */
template <typename... Types, typename... Sizes>
std::tuple<Types*...> allocate_workspace_and_distribute(cudaStream_t stream, GPUMemoryArena::Allocation* alloc, Sizes... sizes) {
	static_assert(sizeof...(Types) == sizeof...(Sizes), "allocate_workspace_and_distribute: one size per type");
	const size_t counts[] = {(size_t)sizes...};
	const size_t total = detail::workspace_bytes<Types...>(std::index_sequence_for<Types...>{}, counts);
	*alloc = allocate_workspace(stream, total);
	return detail::Distribute<Types...>::run(alloc->data(), (size_t)sizes...);
}

TCNN_NAMESPACE_END
