// The host side of a decode burst in one call: the step's tokens go from pinned host memory to
// the device, the instantiated graph of the step is launched `replays` times, and the rows of
// sampled tokens come back to pinned host memory, all on one stream.  The caller does its own
// bookkeeping while the device works and then waits with sb_stream_wait.  (Python reaches the
// same calls one by one through the tensor library; together they cost more than the rest of a
// small step's host work.)
#include <cuda_runtime.h>

extern "C" int sb_graph_burst(void* graph_exec, void* dev_in, const void* host_in, long long in_bytes,
                              int replays, void* host_out, const void* dev_out, long long out_bytes,
                              cudaStream_t stream) {
  cudaError_t e = cudaSuccess;
  if (in_bytes > 0) e = cudaMemcpyAsync(dev_in, host_in, (size_t)in_bytes, cudaMemcpyHostToDevice, stream);
  for (int i = 0; i < replays && e == cudaSuccess; ++i) e = cudaGraphLaunch((cudaGraphExec_t)graph_exec, stream);
  if (e == cudaSuccess && out_bytes > 0)
    e = cudaMemcpyAsync(host_out, dev_out, (size_t)out_bytes, cudaMemcpyDeviceToHost, stream);
  return (int)e;
}

extern "C" int sb_stream_wait(cudaStream_t stream) { return (int)cudaStreamSynchronize(stream); }
