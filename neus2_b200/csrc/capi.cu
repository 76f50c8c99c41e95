// Library-level entry points of libneus2b.so.
#include "common.cuh"

extern "C" const char* neus2b_version(void) { return "neus2b 0.1 (sm_100a)"; }

extern "C" const char* neus2b_error_string(int code) {
	switch (code) {
		case NEUS2B_OK: return "ok";
		case NEUS2B_E_INVALID: return "invalid argument";
		case NEUS2B_E_UNSUPPORTED: return "unsupported configuration";
		case NEUS2B_E_NO_DEVICE: return "no CUDA device";
		case NEUS2B_E_OVERFLOW: return "device-side capacity exceeded";
		case NEUS2B_E_TOO_LARGE: return "request exceeds a compiled-in capacity";
		case NEUS2B_E_IO: return "file could not be opened or written";
		case NEUS2B_E_DEVICE: return "a kernel raised the device error flag";
		case NEUS2B_E_TIMEOUT: return "a bounded wait ran out";
		default: break;
	}
	if (code > 0) return cudaGetErrorString((cudaError_t)code);
	return "unknown error";
}

// Kernel launches issued by this library in this process (every launch site counts itself through N2B_CHECK_LAUNCH).
#include <atomic>
namespace n2b {
static std::atomic<uint64_t> g_launch_count{0};
void count_launch() { g_launch_count.fetch_add(1, std::memory_order_relaxed); }
}  // namespace n2b
extern "C" uint64_t neus2b_launch_count(void) { return n2b::g_launch_count.load(std::memory_order_relaxed); }

// sizeof of every structure that crosses the C ABI, in the order of the header, so that a binding can check its own layout
// against the library it loaded before it passes a pointer.
extern "C" uint32_t neus2b_abi_struct_sizes(uint32_t* sizes, uint32_t capacity) {
	const uint32_t all[] = {(uint32_t)sizeof(neus2b_grid_desc),       (uint32_t)sizeof(neus2b_motion),          (uint32_t)sizeof(neus2b_pcg32),
	                        (uint32_t)sizeof(neus2b_dataset),         (uint32_t)sizeof(neus2b_train_cfg),       (uint32_t)sizeof(neus2b_ray_workspace),
	                        (uint32_t)sizeof(neus2b_adam_cfg),        (uint32_t)sizeof(neus2b_testbed_config),  (uint32_t)sizeof(neus2b_train_stats),
	                        (uint32_t)sizeof(neus2b_render_cfg),      (uint32_t)sizeof(neus2b_render_workspace), (uint32_t)sizeof(neus2b_render_request),
	                        (uint32_t)sizeof(neus2b_training_state)};
	const uint32_t n = (uint32_t)(sizeof(all) / sizeof(all[0]));
	for (uint32_t i = 0; i < n && i < capacity && sizes; ++i) sizes[i] = all[i];
	return n;
}
