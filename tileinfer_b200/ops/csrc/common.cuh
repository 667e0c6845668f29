// Shared device helpers for the sm_100a kernels: bf16 packing, exact int8->bf16 conversion,
// mma.sync fragments for the skinny (M <= 16) products, low-latency peer packets and bounded waits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <utility>

#define TI_HOST_DEVICE __host__ __device__ __forceinline__
#define TI_DEVICE __device__ __forceinline__

namespace ti {

constexpr int kMaxRanks = 8;

// Error bits a kernel may OR into its status word instead of trapping or spinning forever.
enum StatusBits : unsigned {
  kStatusPeerTimeout = 1u,   // a wait on a peer packet / flag ran out of budget
  kStatusBadArgument = 2u,   // a size or alignment precondition did not hold
  kStatusBounds = 4u,        // a checked index was out of range (debug builds)
};

// ---------------------------------------------------------------- checked build
// -DTI_BOUNDS_CHECK: indices derived from run-time data (peer-buffer offsets, KV page numbers, workspace rows) are
// verified before use; a violation sets kStatusBounds in the status word and the access is SKIPPED, so a wrong index
// shows up as an error bit and a wrong result, never as a device fault.  Without the flag the macro is `true` and
// compiles away.  -DTI_JITTER: random delays in front of the packet / flag protocol steps (arrival-order stress).
#ifdef TI_BOUNDS_CHECK
TI_DEVICE bool check_index(long long idx, long long limit, unsigned* status) {
  if (idx >= 0 && idx < limit) return true;
  if (status != nullptr) atomicOr(status, kStatusBounds);
  return false;
}
#define TI_CHECK(idx, limit, status) ti::check_index((long long)(idx), (long long)(limit), (status))
#else
#define TI_CHECK(idx, limit, status) true
#endif
#ifdef TI_JITTER
TI_DEVICE void jitter() {
  unsigned h = (blockIdx.x + 1u) * 2654435761u ^ ((threadIdx.x >> 5) + 1u) * 40503u ^ (unsigned)clock();
  h ^= h >> 13;
  __nanosleep(h % 4000u);
}
#else
TI_DEVICE void jitter() {}
#endif

// ---------------------------------------------------------------- small math
TI_DEVICE float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
TI_DEVICE float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
TI_DEVICE float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }   // 2 ulp: results are rounded to bf16
TI_DEVICE float sigmoid_f(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

TI_DEVICE float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
TI_DEVICE float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
TI_DEVICE uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
TI_DEVICE float bf16_to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
TI_DEVICE float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ---------------------------------------------------------------- int8 -> bf16 (exact)
// `u` holds four offset-binary bytes (s8 ^ 0x80).  Byte i is placed in the mantissa of 2^23, the
// bias 2^23+128 is subtracted (exact in fp32) and the upper halves of two floats are packed: an
// s8 value has at most 8 significant bits, so truncation to bf16 is exact.
TI_DEVICE void cvt_s8x4_bf16x2(uint32_t u, uint32_t& lo01, uint32_t& hi23) {
  const float bias = 8388736.0f;  // 2^23 + 128
  float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - bias;
  float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - bias;
  float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - bias;
  float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - bias;
  lo01 = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
  hi23 = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
}

// ---------------------------------------------------------------- mma.sync m16n8k16 (bf16, fp32 acc)
// Used only for products with at most 16 activation rows (decode GEMV, paged attention), where a
// 128-row tcgen05 tile would be almost empty.
TI_DEVICE void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------- global memory access flavours
TI_DEVICE uint4 ldg_stream16(const void* p) {  // read-once weights: do not keep in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
TI_DEVICE uint4 ldg_cached16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

TI_DEVICE unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------- low-latency peer packets
// A packet is 8 bytes {payload, tag}; an aligned 8-byte store is one transaction, so a reader that
// sees the expected tag also sees the payload.  Two packets are moved with one 16-byte access.
TI_DEVICE void ll_store2(void* dst, float v0, float v1, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"l"(dst), "r"(__float_as_uint(v0)),
               "r"(tag), "r"(__float_as_uint(v1)), "r"(tag)
               : "memory");
}
TI_DEVICE bool ll_try_load2(const void* src, uint32_t tag, float& v0, float& v1) {
  uint32_t a, fa, b, fb;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(a), "=r"(fa), "=r"(b), "=r"(fb)
               : "l"(src)
               : "memory");
  v0 = __uint_as_float(a);
  v1 = __uint_as_float(b);
  return fa == tag && fb == tag;
}
// Waits for a tagged packet pair with a time budget.  On expiry the status word gets
// kStatusPeerTimeout, the payload reads as 0 and the caller carries on (never traps, never hangs).
TI_DEVICE void ll_wait2(const void* src, uint32_t tag, float& v0, float& v1, unsigned long long budget_ns,
                        unsigned* status) {
  if (ll_try_load2(src, tag, v0, v1)) return;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (!ll_try_load2(src, tag, v0, v1)) {
    if ((++spins & 63u) == 0u) {
      if (globaltimer_ns() - t0 > budget_ns) {
        atomicOr(status, kStatusPeerTimeout);
        v0 = 0.f;
        v1 = 0.f;
        return;
      }
    }
  }
}

// Flag wait (acquire at system scope) with the same budget rule.  Returns false on expiry.
TI_DEVICE bool wait_flag_ge(const uint32_t* flag, uint32_t want, unsigned long long budget_ns, unsigned* status) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(flag) : "memory");
  if ((int32_t)(v - want) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (true) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t)(v - want) >= 0) return true;
    if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > budget_ns) {
      atomicOr(status, kStatusPeerTimeout);
      return false;
    }
  }
}
TI_DEVICE void store_flag_release(uint32_t* flag, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(flag), "r"(v) : "memory");
}


// ---------------------------------------------------------------- mbarrier + bulk async copy (TMA engine)
TI_DEVICE uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
TI_DEVICE void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
TI_DEVICE void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
TI_DEVICE void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
TI_DEVICE void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// Linear global -> shared copy by the TMA engine; completion is signalled on `bar` as transferred bytes.
// Both addresses 16-byte aligned, size a multiple of 16.  Source is this GPU's own memory.
TI_DEVICE void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
TI_DEVICE bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on an mbarrier phase.  Returns false (and raises kStatusPeerTimeout) when the budget
// runs out, so a copy that never lands cannot hang the GPU.
TI_DEVICE bool mbar_wait(uint32_t bar, uint32_t parity, unsigned long long budget_ns, unsigned* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > budget_ns) {
      if (status != nullptr) atomicOr(status, kStatusPeerTimeout);
      return false;
    }
  }
  return true;
}


// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-serialization attribute may start while its predecessor in
// the stream is still running; it must call pdl_wait() before it touches anything the predecessor
// writes.  pdl_trigger() lets the successor start.  Kernels use the time before pdl_wait() to prefetch
// data no earlier kernel of the step writes (weights, recurrent state).
TI_DEVICE void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
TI_DEVICE void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

inline int& pdl_enabled() {
  static int flag = [] {
    const char* e = getenv("TI_PDL");
    return e == nullptr ? 1 : atoi(e);
  }();
  return flag;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace ti
