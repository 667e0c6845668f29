// Sampling on the device: logit edits (repetition penalty, logit bias, allow / deny lists, grammar masks) applied to
// the logits in place, and the draw from the gathered top-k candidates (temperature, top-k, top-p, inverse-CDF pick).
//
// Replaces the reference's per-sequence Python loops over GPU logits (engine/model_runner.py:917-974: penalty through
// a Python set, constraints one sequence at a time) and its sampling tail (engine/model_runner.py:1034-1083,
// 1151-1169: torch.topk / softmax / sort / cumsum / multinomial with an `.item()` synchronisation per sequence and a
// broadcast of the chosen ids from rank 0).  Here both kernels sit inside the CUDA-graph decode step: a request with
// a penalty, a bias or a grammar stays on the graph path, and the only device -> host traffic of a step is the chosen
// token id per row plus the communicator's status word, in one small copy.
//
// Every rank runs the same deterministic kernel on the same candidates (already exchanged by the top-k kernel) with
// the same uniform number drawn by the host from a generator all ranks seed alike, so all ranks pick the same token
// without a broadcast.
#include "common.cuh"

namespace ti {

struct EditParams {
  float* logits;            // [M, ld] fp32, this rank's vocabulary shard
  const int* row_slot;      // [M] edit slot of the row, or -1: row untouched
  const float* add_rows;    // [slots, V] value added to every logit (0, a bias, or -inf for a masked token), per slot
  const int* add_valid;     // [slots] 1: the slot's add row is in use
  const int* pen_ids;       // [slots, pen_cap] sorted LOCAL token ids that get the repetition penalty
  const int* pen_cnt;       // [slots]
  const float* pen_rp;      // [slots]
  int M, V, ld, pen_cap, chunk;
};

// grid (M, ceil(V / chunk)): penalty on the listed ids that fall into this block's chunk first (as the reference:
// positive logits are divided by the penalty, the others multiplied), then the additive row.
__global__ void __launch_bounds__(256) logits_edit_kernel(const __grid_constant__ EditParams p) {
  const int m = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const int slot = p.row_slot[m];
  if (slot < 0) return;
  const int lo = blockIdx.y * p.chunk, hi = min(p.V, lo + p.chunk);
  float* row = p.logits + (size_t)m * p.ld;
  const int cnt = min(p.pen_cnt[slot], p.pen_cap);
  if (cnt > 0) {
    const int* ids = p.pen_ids + (size_t)slot * p.pen_cap;
    const float rp = p.pen_rp[slot];
    // first listed id >= lo (the list is sorted)
    int a = 0, b = cnt;
    while (a < b) {
      const int mid = (a + b) >> 1;
      if (ids[mid] < lo) a = mid + 1; else b = mid;
    }
    for (int i = a + threadIdx.x; i < cnt; i += blockDim.x) {
      const int id = ids[i];
      if (id >= hi) break;
      const float v = row[id];
      row[id] = v > 0.f ? v / rp : v * rp;
    }
    __syncthreads();
  }
  if (p.add_valid[slot]) {
    const float* add = p.add_rows + (size_t)slot * p.V;
    for (int n = lo + threadIdx.x; n < hi; n += blockDim.x) row[n] += add[n];
  }
}

struct SampleParams {
  const float* cand_val;    // [M, n_cand]
  const int* cand_idx;      // [M, n_cand] global token ids (-1: empty entry)
  const float* temperature; // [M]  <= 0: greedy
  const int* top_k;         // [M]  <= 0: all candidates
  const float* top_p;       // [M]
  const float* u;           // [M] uniform number in [0, 1)
  int* out_tok;             // [M + 1]: the chosen ids, then a copy of *status_src
  const unsigned* status_src;
  int M, n_cand;
};

constexpr int kMaxCand = 512;

TI_DEVICE bool cand_before(float va, int ia, int pa, float vb, int ib, int pb) {
  // value descending, then token id ascending (empty entries last), then position
  if (va != vb) return va > vb;
  const unsigned ua = (unsigned)ia, ub = (unsigned)ib;   // -1 -> largest
  if (ua != ub) return ua < ub;
  return pa < pb;
}

// One block per row.  Candidates are ranked by counting (n_cand <= 512), then warp 0 runs the distribution.
__global__ void __launch_bounds__(256) sample_kernel(const __grid_constant__ SampleParams p) {
  __shared__ float v_in[kMaxCand], v_s[kMaxCand];
  __shared__ int i_in[kMaxCand], i_s[kMaxCand];
  const int m = blockIdx.x, tid = threadIdx.x, n = p.n_cand;
  pdl_trigger();
  pdl_wait();
  if (m == p.M) {                         // the extra block carries the status word to the host-visible buffer
    if (tid == 0) p.out_tok[p.M] = p.status_src != nullptr ? (int)*p.status_src : 0;
    return;
  }
  for (int i = tid; i < n; i += blockDim.x) {
    v_in[i] = p.cand_val[(size_t)m * n + i];
    i_in[i] = p.cand_idx[(size_t)m * n + i];
  }
  __syncthreads();
  for (int i = tid; i < n; i += blockDim.x) {
    const float v = v_in[i];
    const int id = i_in[i];
    int rank = 0;
    for (int j = 0; j < n; ++j) rank += cand_before(v_in[j], i_in[j], j, v, id, i) ? 1 : 0;
    v_s[rank] = v;
    i_s[rank] = id;
  }
  __syncthreads();
  if (tid >= 32) return;
  const int lane = tid;
  const float temp = p.temperature[m];
  int kk = p.top_k[m];
  if (temp <= 0.f || kk == 1) {
    if (lane == 0) p.out_tok[m] = i_s[0];
    return;
  }
  kk = kk <= 0 ? n : min(kk, n);
  // softmax over the first kk candidates at this temperature (entries of -inf get probability 0)
  const float mx = v_s[0] / temp;
  float z = 0.f;
  for (int i = lane; i < kk; i += 32) {
    const float e = __expf(v_s[i] / temp - mx);
    v_in[i] = e;                                          // reuse as the unnormalised probabilities
    z += e;
  }
  z = warp_sum(z);
  __syncwarp();
  if (lane != 0) return;
  // top-p: the shortest prefix whose probability reaches top_p (an entry is kept while the mass BEFORE it is < top_p)
  const float topp = p.top_p[m];
  float before = 0.f, kept = 0.f;
  int nk = 0;
  for (int i = 0; i < kk; ++i) {
    const float pi = v_in[i] / z;
    if (!(before < topp) || pi <= 0.f) break;
    before += pi;
    kept += pi;
    ++nk;
  }
  nk = max(nk, 1);
  // inverse CDF over the renormalised kept entries: the number of entries whose cumulative mass stays below u
  const float uu = p.u[m];
  float cum = 0.f;
  int pick = 0;
  for (int i = 0; i < nk; ++i) {
    cum += (v_in[i] / z) / kept;
    if (cum < uu) pick = i + 1;
  }
  pick = min(pick, nk - 1);
  p.out_tok[m] = i_s[pick];
}

}  // namespace ti

extern "C" {

int ti_edit_params_size() { return (int)sizeof(ti::EditParams); }
int ti_sample_params_size() { return (int)sizeof(ti::SampleParams); }

int ti_logits_edit(const ti::EditParams* p, void* stream) {
  if (p->M <= 0) return 0;
  if (p->chunk < 256 || p->V < 1) return -2;
  dim3 grid(p->M, (p->V + p->chunk - 1) / p->chunk);
  cudaError_t e = ti::launch_kernel(ti::logits_edit_kernel, grid, dim3(256), 0, (cudaStream_t)stream, true, *p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Chooses one token per row from its candidates; out_tok[M] receives the status word.
int ti_sample(const ti::SampleParams* p, void* stream) {
  if (p->M <= 0) return 0;
  if (p->n_cand < 1 || p->n_cand > ti::kMaxCand) return -2;
  cudaError_t e = ti::launch_kernel(ti::sample_kernel, dim3(p->M + 1), dim3(256), 0, (cudaStream_t)stream, true, *p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // extern "C"
