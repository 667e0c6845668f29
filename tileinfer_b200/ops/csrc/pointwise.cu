// Stand-alone memory-bound ops: embedding gather, RMSNorm, residual+RMSNorm, SiLU*mul, sigmoid*mul.
// In the decode path these are fused into the GEMV prologue/epilogue; the stand-alone forms serve
// the prefill path, TP baselines and tests.  Replaces kernels/rms_norm.py:6-40,
// kernels/residual_rmsnorm.py:7-77 and kernels/act_mul.py:6-115 of the reference (runtime shapes,
// 128-bit accesses, no per-shape recompilation).
#include "common.cuh"

namespace ti {

// h[m, :] = table[ids[m], :]; block 0 also advances the device step counter that tags peer packets.
__global__ void embed_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                             __nv_bfloat16* __restrict__ out, int H, int vocab, unsigned* step) {
  const int m = blockIdx.x;
  long long id = ids[m];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)m * H);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = __ldg(src + c);
  if (step != nullptr && m == 0 && threadIdx.x == 0) *step = *step + 1u;
}

TI_DEVICE float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nw; ++w) t += red[w];
  __syncthreads();
  return t;
}

// y = rmsnorm(x + add?) * (one_plus ? 1 + w : w); optionally also writes the sum r = x + add.
// One block per row; rows of any multiple of 8 elements.
__global__ void rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ add,
                               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                               __nv_bfloat16* __restrict__ r_out, int H, float eps, int one_plus) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* row = reinterpret_cast<float*>(smem);          // [H]
  float* red = row + H;                                  // [32]
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + base + c * 8);
    uint32_t a4[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = bf16lo(a4[i]); f[2 * i + 1] = bf16hi(a4[i]); }
    if (add != nullptr) {
      const uint4 u = *reinterpret_cast<const uint4*>(add + base + c * 8);
      uint32_t b4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // the sum is rounded to bf16 (it becomes the stored residual) before the statistics
        f[2 * i] = round_bf16(f[2 * i] + bf16lo(b4[i]));
        f[2 * i + 1] = round_bf16(f[2 * i + 1] + bf16hi(b4[i]));
      }
      if (r_out != nullptr)
        *reinterpret_cast<uint4*>(r_out + base + c * 8) =
            make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) { row[c * 8 + i] = f[i]; ss += f[i] * f[i]; }
  }
  const float rr = rsqrtf(block_sum(ss, red) / (float)H + eps);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + c * 8));
    uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float w0 = bf16lo(w4[i]) + (one_plus ? 1.f : 0.f), w1 = bf16hi(w4[i]) + (one_plus ? 1.f : 0.f);
      o[i] = pack_bf16(row[c * 8 + 2 * i] * rr * w0, row[c * 8 + 2 * i + 1] * rr * w1);
    }
    *reinterpret_cast<uint4*>(y + base + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// mode 0: out = silu(a) * b     mode 1: out = a * sigmoid(b).  a, b, out: [M, n] with row strides.
__global__ void act_mul_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                               __nv_bfloat16* __restrict__ out, long long total8, int n8, int lda, int ldb, int ldo,
                               int mode) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total8;
       i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / n8;
    const int c = (int)(i - m * n8) * 8;
    const uint4 av = *reinterpret_cast<const uint4*>(a + m * lda + c);
    const uint4 bv = *reinterpret_cast<const uint4*>(b + m * ldb + c);
    uint32_t a4[4] = {av.x, av.y, av.z, av.w}, b4[4] = {bv.x, bv.y, bv.z, bv.w}, o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a0 = bf16lo(a4[j]), a1 = bf16hi(a4[j]), b0 = bf16lo(b4[j]), b1 = bf16hi(b4[j]);
      o[j] = mode == 0 ? pack_bf16(silu_f(a0) * b0, silu_f(a1) * b1) : pack_bf16(a0 * sigmoid_f(b0), a1 * sigmoid_f(b1));
    }
    *reinterpret_cast<uint4*>(out + m * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// gate_up rows are interleaved (g0,u0,g1,u1,...): out[m, j] = silu(gu[m, 2j]) * gu[m, 2j+1]
__global__ void swiglu_interleaved_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                          long long total, int n, int ldg, int ldo) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / n;
    const int j = (int)(i - m * n);
    const uint32_t v = *reinterpret_cast<const uint32_t*>(gu + m * ldg + 2 * j);
    out[m * ldo + j] = __float2bfloat16_rn(silu_f(bf16lo(v)) * bf16hi(v));
  }
}

}  // namespace ti

extern "C" {

int ti_embed(const void* ids, const void* table, void* out, int M, int H, int vocab, void* step, void* stream) {
  if (H % 8) return -2;
  ti::embed_kernel<<<M, 128, 0, (cudaStream_t)stream>>>((const long long*)ids, (const __nv_bfloat16*)table,
                                                        (__nv_bfloat16*)out, H, vocab, (unsigned*)step);
  return (int)cudaGetLastError();
}

int ti_rmsnorm(const void* x, const void* add, const void* w, void* y, void* r_out, int M, int H, float eps,
               int one_plus, void* stream) {
  if (H % 8 || H > 12288) return -2;
  const size_t sm = (size_t)H * 4 + 32 * 4;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(ti::rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 12288 * 4 + 128);
    attr = true;
  }
  const int threads = H >= 2048 ? 256 : 64;
  ti::rmsnorm_kernel<<<M, threads, sm, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)add,
                                                               (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
                                                               (__nv_bfloat16*)r_out, H, eps, one_plus);
  return (int)cudaGetLastError();
}

int ti_act_mul(const void* a, const void* b, void* out, int M, int n, int lda, int ldb, int ldo, int mode,
               void* stream) {
  if (n % 8 || lda % 8 || ldb % 8 || ldo % 8) return -2;
  const long long total8 = (long long)M * (n / 8);
  const int blocks = (int)min((long long)148 * 8, (total8 + 255) / 256);
  ti::act_mul_kernel<<<max(blocks, 1), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, total8, n / 8, lda, ldb, ldo, mode);
  return (int)cudaGetLastError();
}

int ti_swiglu_interleaved(const void* gu, void* out, int M, int n, int ldg, int ldo, void* stream) {
  const long long total = (long long)M * n;
  const int blocks = (int)min((long long)148 * 8, (total + 255) / 256);
  ti::swiglu_interleaved_kernel<<<max(blocks, 1), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total, n, ldg, ldo);
  return (int)cudaGetLastError();
}

}  // extern "C"
