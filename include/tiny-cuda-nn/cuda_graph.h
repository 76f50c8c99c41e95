/* tiny-cuda-nn/cuda_graph.h of the B200-native stand-in: capture a stream's launches once, replay them as one graph
 * launch afterwards (launch-bound inner loops).  Included by include/neural-graphics-primitives/testbed.h:20.
 *
 *   CudaGraph g;
 *   { auto guard = g.capture_guard(stream);  ... launches on stream ...  }   // first time: captured, then launched;
 *                                                                            // later: re-captured and updated in place
 * Synchronising calls inside the guarded region end the capture with an error; call g.schedule_synchronize() there
 * instead and the guard synchronises after the replay. */
#pragma once
#include <tiny-cuda-nn/common.h>

#include <deque>

TCNN_NAMESPACE_BEGIN

class CudaGraph;
inline std::deque<CudaGraph*>& current_captures() {
	static thread_local std::deque<CudaGraph*> s_current;
	return s_current;
}
inline CudaGraph* current_capture() { return current_captures().empty() ? nullptr : current_captures().front(); }

class CudaGraph {
public:
	CudaGraph() = default;
	~CudaGraph() {
		try {
			reset();
		} catch (const std::exception& e) {
			if (std::string{e.what()}.find("driver shutting down") == std::string::npos) std::cerr << "Could not destroy cuda graph: " << e.what() << std::endl;
		}
	}
	CudaGraph(const CudaGraph&) = delete;
	CudaGraph& operator=(const CudaGraph&) = delete;
	CudaGraph& operator=(CudaGraph&& other) {
		std::swap(m_graph, other.m_graph);
		std::swap(m_graph_instance, other.m_graph_instance);
		std::swap(m_synchronize_when_capture_done, other.m_synchronize_when_capture_done);
		return *this;
	}
	CudaGraph(CudaGraph&& other) { *this = std::move(other); }

	ScopeGuard capture_guard(cudaStream_t stream) {
		/* no nested captures: an outer capture already records these launches */
		if (stream == nullptr || stream == cudaStreamLegacy) return ScopeGuard{};
		cudaStreamCaptureStatus status;
		CUDA_CHECK_THROW(cudaStreamIsCapturing(stream, &status));
		if (status != cudaStreamCaptureStatusNone) return ScopeGuard{};
		cudaError_t err = cudaStreamIsCapturing(cudaStreamLegacy, &status);
		if (err == cudaErrorStreamCaptureImplicit) {
			cudaGetLastError();
			return ScopeGuard{};
		}
		if (status != cudaStreamCaptureStatusNone) return ScopeGuard{};

		if (m_graph) {
			CUDA_CHECK_THROW(cudaGraphDestroy(m_graph));
			m_graph = nullptr;
		}
		CUDA_CHECK_THROW(cudaStreamBeginCapture(stream, cudaStreamCaptureModeRelaxed));
		current_captures().push_front(this);

		return ScopeGuard{[this, stream]() {
			CUDA_CHECK_THROW(cudaStreamEndCapture(stream, &m_graph));
			if (current_captures().front() != this) throw std::runtime_error("CudaGraph: captures must end in the reverse order of their start");
			current_captures().pop_front();
			if (m_synchronize_when_capture_done) {
				CUDA_CHECK_THROW(cudaDeviceSynchronize());
				m_synchronize_when_capture_done = false;
			}
			if (!m_graph) {
				if (m_graph_instance) CUDA_CHECK_THROW(cudaGraphExecDestroy(m_graph_instance));
				m_graph_instance = nullptr;
				return;
			}
			if (m_graph_instance) {
				cudaGraphExecUpdateResultInfo info;
				if (cudaGraphExecUpdate(m_graph_instance, m_graph, &info) != cudaSuccess) {
					cudaGetLastError(); /* topology changed: instantiate anew */
					CUDA_CHECK_THROW(cudaGraphExecDestroy(m_graph_instance));
					m_graph_instance = nullptr;
				}
			}
			if (!m_graph_instance) CUDA_CHECK_THROW(cudaGraphInstantiate(&m_graph_instance, m_graph, 0));
			CUDA_CHECK_THROW(cudaGraphLaunch(m_graph_instance, stream));
		}};
	}
	void reset() {
		if (m_graph) {
			CUDA_CHECK_THROW(cudaGraphDestroy(m_graph));
			m_graph = nullptr;
		}
		if (m_graph_instance) {
			CUDA_CHECK_THROW(cudaGraphExecDestroy(m_graph_instance));
			m_graph_instance = nullptr;
		}
	}
	void schedule_synchronize() { m_synchronize_when_capture_done = true; }

private:
	cudaGraph_t m_graph = nullptr;
	cudaGraphExec_t m_graph_instance = nullptr;
	bool m_synchronize_when_capture_done = false;
};

TCNN_NAMESPACE_END
