// CUDA graphs on the runtime API, for the step function's decode graphs: begin and end a stream capture, instantiate,
// launch, destroy. The reference replays one graph per decode token the same way (engine/models/lfm2_moe/engine.py:745-794).
//
// Why not torch.cuda.CUDAGraph: measured on a B200 with torch 2.11, from the fourth capture_begin/capture_end of that class
// in a process on, every graph of the process replays about 5 % slower (a decode step of 190 small kernels: 1115 -> 1178 us
// on the device; the host's launch takes 4 us either way), empty captures and captures that are never instantiated
// included, and it stays so after the graphs are destroyed. Captures made with these calls, with torch's allocator
// pointed at a memory pool of its own meanwhile (torch.cuda.use_mem_pool), do not show it at any number of graphs.
#include "common.cuh"

using namespace tl;

// Capture mode: calls that are unsafe during a capture (an allocation by the caching allocator that has to reach the
// driver) are this thread's own and belong to the capture, so only other threads' captures are protected.
extern "C" int tl_graph_capture_begin(cudaStream_t stream) {
  return (int)cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
}

// Ends the capture on `stream` and instantiates what was captured; *exec receives the executable graph (null on failure)
// and *nodes the number of its nodes. The captured graph itself is destroyed.
extern "C" int tl_graph_capture_end(cudaStream_t stream, void** exec, int* nodes) {
  *exec = nullptr;
  if (nodes) *nodes = 0;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(stream, &graph);
  if (e != cudaSuccess) {
    if (graph) cudaGraphDestroy(graph);
    return (int)e;
  }
  TL_REQUIRE(graph != nullptr, "graph capture: the stream was not capturing (%d)", 0);
  size_t n = 0;
  e = cudaGraphGetNodes(graph, nullptr, &n);
  if (e == cudaSuccess && nodes) *nodes = (int)n;
  cudaGraphExec_t ex = nullptr;
  if (e == cudaSuccess) e = cudaGraphInstantiate(&ex, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return (int)e;
  *exec = (void*)ex;
  return 0;
}

extern "C" int tl_graph_launch(void* exec, cudaStream_t stream) {
  TL_REQUIRE(exec != nullptr, "graph launch: no graph (%d)", 0);
  return (int)cudaGraphLaunch((cudaGraphExec_t)exec, stream);
}

extern "C" int tl_graph_destroy(void* exec) {
  if (!exec) return 0;
  return (int)cudaGraphExecDestroy((cudaGraphExec_t)exec);
}
