// Row-parallel products with many rows (prefill chunks, large decode batches) under tensor parallelism:
// all-reduce + residual add + RMSNorm + activation quantisation in ONE kernel, the partial sums read straight out of
// every rank's symmetric buffer over NVLink (in-switch reduction with multimem.ld_reduce where the buffers are bound
// to an NVLS multicast object, plain peer loads otherwise).
//
// Replaces the reference's prefill sequence GEMM -> NCCL all_reduce(async) -> wait -> residual_rmsnorm kernel
// (model/qwen_36.py:680-690, 701-708, 1087-1097, 1119-1125) and this package's own baseline of tcgen05 GEMM ->
// NCCL all-reduce -> add.  Data flow of one row-parallel product:
//
//   tcgen05 GEMM          epilogue stores this rank's partial tile, bf16, directly into its symmetric buffer
//                         (two buffers alternate by the collective's position in the step);
//   ar_rows_kernel        block 0 publishes "my partials are complete" (one tagged flag per peer, release at system
//                         scope); every block waits, bounded, for the flags of all ranks, then owns one row: sum of the
//                         tp partial rows (fp32) + residual -> the new residual stream row (bf16, local), and, still in
//                         registers, the prologue of the CONSUMING product: RMSNorm(1+w) and either the two int8 limb
//                         planes + row scale (W8A16 GEMM) or the normalised bf16 row (bf16 GEMM).
//
// Two-shot form for many rows on four or more ranks (two_shot = 1): in the one-shot form every GPU serves each of its
// partial rows to all tp requesters (tp x M x N x 2 bytes of NVLink egress per product); here rank r first reduces only
// the rows m = r (mod tp) and writes the bf16 sums back over that row in EVERY rank's partial buffer (multimem.st
// through the switch, or peer stores), the last block to finish publishes a second flag, and the row kernel then
// reads the sums from LOCAL memory.  A row is read by its owner alone before the owner overwrites it, so the
// exchange is in place; per GPU M x N x 2 bytes leave and arrive once, whatever tp is.
//
// Every rank reduces every row itself (one-shot): nothing is written to a peer but flags, so there is no second
// barrier and no remote store to order; a row crosses NVLink tp-1 times per rank (10 KB per row at N = 5120), a few
// percent of the time of the GEMM that produced it.  Tags come from the device step counter and the collective's
// position, so CUDA-graph replays need no host patching.  The flag wait is bounded: on expiry the status word is
// set and the kernel carries on with whatever the buffers hold (never traps, never hangs).
#include "common.cuh"

namespace ti {

struct ArRowsParams {
  uint64_t part_peer[kMaxRanks];   // every rank's partial buffer [M, N] bf16 as mapped in this process
  uint64_t part_mc;                // multicast address of the same buffer, or 0: plain peer loads
  uint64_t flag_peer[kMaxRanks];   // every rank's flag array [kMaxRanks] (uint32) as mapped in this process
  const __nv_bfloat16* resid;      // [M, N] local, or nullptr
  __nv_bfloat16* h_out;            // [M, N] local: resid + sum over ranks
  const __nv_bfloat16* norm_w;     // [N] RMSNorm weight (1+w convention), or nullptr: no normalisation
  int8_t* xh;                      // mode 1: limb planes [M, N] and row scales [M]
  uint8_t* xl;
  float* xscale;
  __nv_bfloat16* xn;               // mode 2: normalised bf16 rows [M, N]
  const unsigned* step_ptr;
  unsigned* status;
  unsigned long long timeout_ns;
  int M, N, tp, rank, order, mode;
  float eps;
  int rows_cap;                    // rows the partial buffers hold (checked builds; 0: unknown)
  int two_shot;                    // 1: reduce-scatter + broadcast first (ar_reduce_bcast_kernel), the row kernel reads local sums
                                   // (2 / 3: only the first / second of the two launches)
};

constexpr int kFlagRound2 = kMaxRanks;          // flag slots of the second round (one per source rank)
constexpr int kFlagCounter = 2 * kMaxRanks;     // this rank's count of finished blocks of the reduce kernel

TI_DEVICE uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Sum over all ranks of the 16 bytes (8 bf16) at this offset of the multicast window, accumulated in fp32 by the switch.
TI_DEVICE uint4 multimem_ld_reduce_bf16x8(uint64_t mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

// The same 16 bytes stored into every rank's copy of the multicast window.
TI_DEVICE void multimem_st_bf16x8(uint64_t mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1,%2,%3,%4};\n" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
TI_DEVICE void st_volatile16(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// First shot of the two-shot form: block b owns row m = b * tp + rank.
template <bool MC>
__global__ void __launch_bounds__(512) ar_reduce_bcast_kernel(const __grid_constant__ ArRowsParams p) {
  __shared__ int s_last;
  const int tid = threadIdx.x;
  const int m = blockIdx.x * p.tp + p.rank;
  const unsigned tag = (*p.step_ptr) * 65536u + (unsigned)p.order + 1u;
  pdl_trigger();
  pdl_wait();                                  // the producing GEMM has completed: this rank's partials are in memory
  if (blockIdx.x == 0 && tid == 0) {
    jitter();
    __threadfence_system();
    for (int q = 0; q < p.tp; ++q)
      store_flag_release(reinterpret_cast<uint32_t*>(p.flag_peer[q]) + p.rank, tag);
  }
  if (tid < p.tp) {
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.flag_peer[p.rank]);
    wait_flag_ge(mine + tid, tag, p.timeout_ns, p.status);
  }
  __syncthreads();
  if (m < p.M && (p.rows_cap <= 0 || TI_CHECK(m, p.rows_cap, p.status))) {
    const int nchunk = p.N >> 3;
    const size_t row_off = (size_t)m * p.N * 2;
    for (int c = tid; c < nchunk; c += 512) {
      const size_t off = row_off + (size_t)c * 16;
      if (MC) {
        multimem_st_bf16x8(p.part_mc + off, multimem_ld_reduce_bf16x8(p.part_mc + off));
      } else {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
        uint4 q[kMaxRanks];                      // all ranks' loads in flight together, summed in rank order
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          q[r] = r < p.tp ? ld_volatile16(reinterpret_cast<const uint8_t*>(p.part_peer[r]) + off) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
          const uint32_t w4[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) { v[2 * i] += bf16lo(w4[i]); v[2 * i + 1] += bf16hi(w4[i]); }
        }
        const uint4 o = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        for (int r = 0; r < p.tp; ++r) st_volatile16(reinterpret_cast<uint8_t*>(p.part_peer[r]) + off, o);
      }
    }
  }
  // every thread's stores are visible system-wide before this block is counted; the last block publishes the second flag
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    unsigned* counter = reinterpret_cast<unsigned*>(p.flag_peer[p.rank]) + kFlagCounter;
    const unsigned prev = atomicAdd(counter, 1u);
    s_last = prev + 1 == gridDim.x;
    if (s_last) {
      *counter = 0;                              // ready for the next launch (launches of one rank are stream-ordered)
      __threadfence_system();
      jitter();
      for (int q = 0; q < p.tp; ++q)
        store_flag_release(reinterpret_cast<uint32_t*>(p.flag_peer[q]) + kFlagRound2 + p.rank, tag);
    }
  }
}

template <bool MC>
__global__ void __launch_bounds__(512) ar_rows_kernel(const __grid_constant__ ArRowsParams p) {
  __shared__ float red[16], red2[16];
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned tag = (*p.step_ptr) * 65536u + (unsigned)p.order + 1u;
  pdl_trigger();
  pdl_wait();                                  // the producing GEMM has completed: this rank's partials are in memory
  if (!p.two_shot && m == 0 && tid == 0) {
    jitter();
    __threadfence_system();
    for (int q = 0; q < p.tp; ++q)
      store_flag_release(reinterpret_cast<uint32_t*>(p.flag_peer[q]) + p.rank, tag);
  }
  if (tid < p.tp) {                            // two-shot: every rank has broadcast the sums of its rows (second flag round)
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.flag_peer[p.rank]) + (p.two_shot ? kFlagRound2 : 0);
    wait_flag_ge(mine + tid, tag, p.timeout_ns, p.status);
  }
  __syncthreads();

  const int nchunk = p.N >> 3;
  const size_t row_off = (size_t)m * p.N * 2;
  if (p.rows_cap > 0 && !TI_CHECK(m, p.rows_cap, p.status)) return;
  float v[5][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 5; ++j) {
    const int c = tid + j * 512;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[j][i] = 0.f;
    if (c < nchunk) {
      const size_t off = row_off + (size_t)c * 16;
      if (MC) {
        const uint4 q = multimem_ld_reduce_bf16x8(p.part_mc + off);
        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { v[j][2 * i] = bf16lo(w4[i]); v[j][2 * i + 1] = bf16hi(w4[i]); }
      } else {
        const int r0 = p.two_shot ? p.rank : 0, r1 = p.two_shot ? p.rank + 1 : p.tp;     // two-shot: the sums are local
        uint4 q[kMaxRanks];                    // all ranks' loads in flight together; rank order: bit-identical sums everywhere
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          q[r] = (r >= r0 && r < r1) ? ld_volatile16(reinterpret_cast<const uint8_t*>(p.part_peer[r]) + off) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
          const uint32_t w4[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) { v[j][2 * i] += bf16lo(w4[i]); v[j][2 * i + 1] += bf16hi(w4[i]); }
        }
      }
      uint32_t o4[4];
      uint4 rq = make_uint4(0, 0, 0, 0);
      if (p.resid != nullptr) rq = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.resid) + off);
      const uint32_t r4[4] = {rq.x, rq.y, rq.z, rq.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // the sum is rounded to bf16: it IS the stored residual stream, statistics follow the stored values
        v[j][2 * i] = round_bf16(v[j][2 * i] + bf16lo(r4[i]));
        v[j][2 * i + 1] = round_bf16(v[j][2 * i + 1] + bf16hi(r4[i]));
        o4[i] = pack_bf16(v[j][2 * i], v[j][2 * i + 1]);
        ss += v[j][2 * i] * v[j][2 * i] + v[j][2 * i + 1] * v[j][2 * i + 1];
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.h_out) + off) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
    }
  }
  if (p.mode == 0) return;
  // ---- prologue of the consuming product: RMSNorm(1 + w), then limbs or bf16
  if (p.norm_w != nullptr) {
    uint4 nwv[5];
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      const int c = tid + j * 512;
      nwv[j] = c < nchunk ? *reinterpret_cast<const uint4*>(p.norm_w + (size_t)c * 8) : make_uint4(0, 0, 0, 0);
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 16; ++w) tot += red[w];
    const float rr = rsqrtf(tot / (float)p.N + p.eps);
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      const uint32_t n4[4] = {nwv[j].x, nwv[j].y, nwv[j].z, nwv[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[j][2 * i] = round_bf16(v[j][2 * i] * rr * (1.f + bf16lo(n4[i])));
        v[j][2 * i + 1] = round_bf16(v[j][2 * i + 1] * rr * (1.f + bf16hi(n4[i])));
      }
    }
  }
  if (p.mode == 2) {
#pragma unroll
    for (int j = 0; j < 5; ++j) {
      const int c = tid + j * 512;
      if (c >= nchunk) continue;
      *reinterpret_cast<uint4*>(p.xn + (size_t)m * p.N + (size_t)c * 8) =
          make_uint4(pack_bf16(v[j][0], v[j][1]), pack_bf16(v[j][2], v[j][3]), pack_bf16(v[j][4], v[j][5]), pack_bf16(v[j][6], v[j][7]));
    }
    return;
  }
  float mx = 0.f;
#pragma unroll
  for (int j = 0; j < 5; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(v[j][i]));
  mx = warp_max(mx);
  if (lane == 0) red2[warp] = mx;
  __syncthreads();
  float a = 0.f;
#pragma unroll
  for (int w = 0; w < 16; ++w) a = fmaxf(a, red2[w]);
  int e = (int)((__float_as_uint(a) >> 23) & 0xffu) - 127;
  e = max(e, -100);
  if (!(a < 3.0e38f)) e = 127;
  const float qs = exp2f((float)(14 - e));
  if (tid == 0) p.xscale[m] = exp2f((float)(e - 14));
#pragma unroll
  for (int j = 0; j < 5; ++j) {
    const int c = tid + j * 512;
    if (c >= nchunk) continue;
    uint32_t hw[2] = {0, 0}, lw[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = max(-32768, min(32767, __float2int_rn(v[j][i] * qs)));
      hw[i >> 2] |= (uint32_t)((q >> 8) & 0xff) << (8 * (i & 3));
      lw[i >> 2] |= (uint32_t)(q & 0xff) << (8 * (i & 3));
    }
    *reinterpret_cast<uint2*>(p.xh + (size_t)m * p.N + (size_t)c * 8) = make_uint2(hw[0], hw[1]);
    *reinterpret_cast<uint2*>(p.xl + (size_t)m * p.N + (size_t)c * 8) = make_uint2(lw[0], lw[1]);
  }
}

}  // namespace ti

extern "C" {

int ti_ar_rows_params_size() { return (int)sizeof(ti::ArRowsParams); }

// One block per row.  mode 0: h_out only; 1: + limb planes of RMSNorm(h_out); 2: + normalised bf16 rows.
int ti_ar_rows(const ti::ArRowsParams* p, void* stream) {
  if (p->M <= 0) return 0;
  if (p->N % 8 || p->N > 512 * 5 * 8 || p->tp < 1 || p->tp > ti::kMaxRanks || p->mode < 0 || p->mode > 2) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (p->two_shot && p->tp > 1) {
    // two_shot 1: both shots; 2 / 3: only the first / the second (ranks emulated one after the other on one GPU)
    const dim3 g1((p->M + p->tp - 1) / p->tp);
    e = cudaSuccess;
    if (p->two_shot != 3) {
      if (p->part_mc != 0) e = ti::launch_kernel(ti::ar_reduce_bcast_kernel<true>, g1, dim3(512), 0, st, true, *p);
      else e = ti::launch_kernel(ti::ar_reduce_bcast_kernel<false>, g1, dim3(512), 0, st, true, *p);
      if (e != cudaSuccess) return (int)e;
    }
    if (p->two_shot != 2) e = ti::launch_kernel(ti::ar_rows_kernel<false>, dim3(p->M), dim3(512), 0, st, true, *p);   // sums are local now
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
  }
  if (p->part_mc != 0) e = ti::launch_kernel(ti::ar_rows_kernel<true>, dim3(p->M), dim3(512), 0, st, true, *p);
  else e = ti::launch_kernel(ti::ar_rows_kernel<false>, dim3(p->M), dim3(512), 0, st, true, *p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // extern "C"
