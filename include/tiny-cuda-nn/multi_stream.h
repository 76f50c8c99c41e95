/* tiny-cuda-nn/multi_stream.h of the B200-native stand-in: helper streams that fork from and join a parent stream through
 * events, so that independent pieces of a step overlap without a host synchronisation.  Included by
 * include/neural-graphics-primitives/testbed.h:24 and transform_network.h:12. */
#pragma once
#include <tiny-cuda-nn/common.h>

#include <unordered_map>

TCNN_NAMESPACE_BEGIN

/* a stream and an event recorded on it */
class StreamAndEvent {
public:
	StreamAndEvent() {
		CUDA_CHECK_THROW(cudaStreamCreateWithFlags(&m_stream, cudaStreamNonBlocking));
		CUDA_CHECK_THROW(cudaEventCreateWithFlags(&m_event, cudaEventDisableTiming));
	}
	~StreamAndEvent() {
		if (m_stream) cudaStreamDestroy(m_stream);
		if (m_event) cudaEventDestroy(m_event);
	}
	StreamAndEvent(const StreamAndEvent&) = delete;
	StreamAndEvent& operator=(const StreamAndEvent&) = delete;
	StreamAndEvent& operator=(StreamAndEvent&& other) {
		std::swap(m_stream, other.m_stream);
		std::swap(m_event, other.m_event);
		return *this;
	}
	StreamAndEvent(StreamAndEvent&& other) { *this = std::move(other); }

	/* work queued on this stream from now on starts after what `stream` holds now */
	void wait_for(cudaStream_t stream) {
		cudaEvent_t e;
		CUDA_CHECK_THROW(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
		CUDA_CHECK_THROW(cudaEventRecord(e, stream));
		CUDA_CHECK_THROW(cudaStreamWaitEvent(m_stream, e, 0));
		CUDA_CHECK_THROW(cudaEventDestroy(e));
	}
	/* `stream` waits for what this stream holds now */
	void signal(cudaStream_t stream) {
		CUDA_CHECK_THROW(cudaEventRecord(m_event, m_stream));
		CUDA_CHECK_THROW(cudaStreamWaitEvent(stream, m_event, 0));
	}
	cudaStream_t get() { return m_stream; }

private:
	cudaStream_t m_stream = {};
	cudaEvent_t m_event = {};
};

/* n helper streams attached to a parent */
class MultiStream {
public:
	MultiStream() { CUDA_CHECK_THROW(cudaEventCreateWithFlags(&m_event, cudaEventDisableTiming)); }
	~MultiStream() { cudaEventDestroy(m_event); }
	MultiStream(const MultiStream&) = delete;
	MultiStream& operator=(const MultiStream&) = delete;

	void resize(size_t n_streams) {
		if (n_streams > m_streams.size()) m_streams.resize(n_streams);
	}
	size_t size() const { return m_streams.size(); }
	void wait_for(cudaStream_t stream) {
		if (m_streams.empty()) return;
		CUDA_CHECK_THROW(cudaEventRecord(m_event, stream));
		for (auto& s : m_streams) CUDA_CHECK_THROW(cudaStreamWaitEvent(s.get(), m_event, 0));
	}
	void signal(cudaStream_t stream) {
		for (auto& s : m_streams) s.signal(stream);
	}
	cudaStream_t get(size_t idx) {
		if (idx >= m_streams.size()) throw std::runtime_error("MultiStream: stream index out of range");
		return m_streams.at(idx).get();
	}

private:
	std::vector<StreamAndEvent> m_streams;
	cudaEvent_t m_event = {};
};

/* helpers that start after the parent's queued work on construction and that the parent waits for on destruction */
class SyncedMultiStream {
public:
	SyncedMultiStream() = default;
	SyncedMultiStream(cudaStream_t stream, size_t n_streams) : m_main_stream{stream}, m_n_streams{n_streams} {
		if (m_n_streams == 0) throw std::runtime_error("SyncedMultiStream: needs at least one stream");
		if (m_n_streams == 1) return; /* stream 0 is the parent itself */
		m_multi_stream = &helper_streams(stream);
		m_multi_stream->resize(m_n_streams - 1);
		m_multi_stream->wait_for(m_main_stream);
	}
	~SyncedMultiStream() {
		if (m_multi_stream) m_multi_stream->signal(m_main_stream);
	}
	SyncedMultiStream(const SyncedMultiStream&) = delete;
	SyncedMultiStream& operator=(const SyncedMultiStream&) = delete;
	SyncedMultiStream& operator=(SyncedMultiStream&& other) {
		std::swap(m_multi_stream, other.m_multi_stream);
		std::swap(m_main_stream, other.m_main_stream);
		std::swap(m_n_streams, other.m_n_streams);
		return *this;
	}
	SyncedMultiStream(SyncedMultiStream&& other) { *this = std::move(other); }

	cudaStream_t get(size_t idx) {
		if (m_n_streams == 0) throw std::runtime_error("SyncedMultiStream: empty");
		if (idx == 0) return m_main_stream;
		if (!m_multi_stream) throw std::runtime_error("SyncedMultiStream: stream index out of range");
		return m_multi_stream->get(idx - 1);
	}

private:
	static MultiStream& helper_streams(cudaStream_t parent) {
		static std::unordered_map<cudaStream_t, std::unique_ptr<MultiStream>> s_helpers;
		auto& h = s_helpers[parent];
		if (!h) h = std::make_unique<MultiStream>();
		return *h;
	}
	MultiStream* m_multi_stream = nullptr;
	cudaStream_t m_main_stream = {};
	size_t m_n_streams = 0;
};

TCNN_NAMESPACE_END
