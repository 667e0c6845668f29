// Peer-memory plumbing for the fused tensor-parallel kernels: device allocations that other ranks of
// the node map through CUDA IPC, and a bounded-wait probe.
//
// The reference has no counterpart: it reaches its peers only through NCCL collectives
// (engine/parallel.py:98-200).  Here each rank allocates its packet buffers with cudaMalloc, hands
// the IPC handle to the other ranks over the torch.distributed store, and every rank maps all of them.
// Kernels then store into / poll those mappings directly over NVLink.
#include "common.cuh"

namespace ti {

__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t want, unsigned long long budget_ns,
                                 unsigned* status, unsigned* result) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *result = wait_flag_ge(flag, want, budget_ns, status) ? 1u : 0u;
}

}  // namespace ti

extern "C" {

int ti_symm_alloc(void** out, size_t bytes) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, bytes);
}

int ti_symm_free(void* p) { return (int)cudaFree(p); }

int ti_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }

int ti_ipc_get_handle(void* dptr, void* handle_out) {
  return (int)cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle_out), dptr);
}

int ti_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}

int ti_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

int ti_memset_async(void* p, int value, size_t bytes, void* stream) {
  return (int)cudaMemsetAsync(p, value, bytes, (cudaStream_t)stream);
}

// Waits (bounded by budget_ns) for *flag >= want on the device; result = 1 if seen, 0 on expiry, in
// which case kStatusPeerTimeout is OR-ed into *status.  The context stays usable either way.
int ti_wait_flag_probe(const void* flag, unsigned want, unsigned long long budget_ns, void* status, void* result,
                       void* stream) {
  ti::wait_flag_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const uint32_t*)flag, want, budget_ns,
                                                          (unsigned*)status, (unsigned*)result);
  return (int)cudaGetLastError();
}

}  // extern "C"
