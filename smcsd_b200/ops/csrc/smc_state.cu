// Device-side SMC bookkeeping, free of host synchronisation so the whole cycle fits in one graph:
//   prepare_cycle   pop (gamma+1) pages per active row from the device free stack, extend the block
//                   table, advance lengths, emit the cycle inputs (incl. the live S-1 page lookup)
//   write_back      token history, finish detection (length / EOS), float64 weight accumulation
//   collect         per group: softmax of interval weights, ESS test, systematic resampling with a
//                   Philox offset, (dst, src) job list, logZ update, weight reset
//   resample_apply  per job: release dst pages (pages reaching zero go back on the free stack),
//                   share src pages (+1 ref), copy lineage scalars and token history
//   state_copy      per job: copy recurrent (GDN) state rows src -> dst for every layer
#include "common.cuh"

namespace smc {

constexpr int MAX_EOS = 8;

struct SlotArrays {
  int* seq_lens;
  int* verified_ids;
  int* prev_ids;
  int* token_counts;
  uint8_t* finished;
  int* finished_len;
  int* finish_code;
  int* matched_eos;
  const uint8_t* ignore_eos;
  const int* max_new_tokens;
  const int* eos_ids;          // [slots, MAX_EOS]
  double* log_weights;
  double* interval_weights;
  int* all_token_ids;          // [slots, max_out]
  int max_out;
  int* block_table;            // [rows, bt_stride]
  int bt_stride;
  int* refcount;
  int* free_stack;
  int* free_count;
  int* alloc_error;
  int n_pages;
};

// Per-cycle device buffers filled by the prologue and read by the forwards of one cycle.
struct CycleIO {
  int* orig_seq;          // [bs] S at cycle start
  int* x0;                // [bs]
  int* prev;              // [bs]
  int* cache_locs;        // [bs, G]
  int* positions_verify;  // [bs, G] = S + j
  int* step_pos;          // [G, bs]  position (and prefix length) of single-token draft step j
  int* step_locs;         // [G, bs]
  int* head_ids;          // [bs, 2] = prev, x0
  int* head_pos;          // [bs, 2] = S-1, S
  int* head_locs;         // [bs, 2] = page of S-1 (looked up live), fresh page of S
  int* head_prefix;       // [bs]    = S-1
  int* verify_ids;        // [bs, G] = x0, d0..d_{gamma-1}   (assembled after the draft phase)
  int* verify_given;      // [bs, G] = d0..d_{gamma-1}, -1    (tokens to score; -1 = sample the bonus)
};

// counters: [0] cycle step, [1] resample jobs of this cycle, [2] groups resampled so far
__global__ void prepare_cycle_kernel(SlotArrays a, const int* __restrict__ active, int bs, int G,
                                     long long* __restrict__ counters, CycleIO io) {
  __shared__ int s_base;
  const int total = bs * G;
  if (threadIdx.x == 0) {
    const int cnt = *a.free_count;
    if (cnt >= total) {
      s_base = cnt - total;
      *a.free_count = cnt - total;
    } else {
      s_base = -1;
      atomicOr(a.alloc_error, SMC_ERR_ALLOC_EXHAUSTED);
    }
    counters[0] += 1;
    counters[1] = 0;
  }
  __syncthreads();
  const int base = s_base;
  for (int t = threadIdx.x; t < total; t += blockDim.x) {
    const int b = t / G, j = t % G;
    const int slot = active[b];
    const int S = a.seq_lens[slot];
    int page = 0;
    if (base >= 0) {
      page = a.free_stack[base + t];
      a.refcount[page] = 1;
    }
    if (S + j < a.bt_stride) a.block_table[(size_t)slot * a.bt_stride + S + j] = page;
    else atomicOr(a.alloc_error, SMC_ERR_BOUNDS);
    io.cache_locs[t] = page;
    io.positions_verify[t] = S + j;
    io.step_pos[j * bs + b] = S + j;
    io.step_locs[j * bs + b] = page;
    if (j == 0) {
      const int xv = a.verified_ids[slot], pv = a.prev_ids[slot];
      const int ploc = S > 0 ? a.block_table[(size_t)slot * a.bt_stride + S - 1] : 0;
      io.orig_seq[b] = S;
      io.x0[b] = xv;
      io.prev[b] = pv;
      io.head_ids[2 * b] = pv;
      io.head_ids[2 * b + 1] = xv;
      io.head_pos[2 * b] = S > 0 ? S - 1 : 0;
      io.head_pos[2 * b + 1] = S;
      io.head_locs[2 * b] = ploc;
      io.head_locs[2 * b + 1] = page;
      io.head_prefix[b] = S > 0 ? S - 1 : 0;
    }
  }
  __syncthreads();
  for (int b = threadIdx.x; b < bs; b += blockDim.x) a.seq_lens[active[b]] += G;
}

// drafts [gamma, bs] step-major -> verify_ids / verify_given [bs, G]
__global__ void assemble_verify_kernel(CycleIO io, const int* __restrict__ drafts, int bs, int gamma) {
  const int G = gamma + 1;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < bs * G; t += gridDim.x * blockDim.x) {
    const int b = t / G, k = t % G;
    io.verify_ids[t] = k == 0 ? io.x0[b] : drafts[(k - 1) * bs + b];
    io.verify_given[t] = k < gamma ? drafts[k * bs + b] : -1;
  }
}

// drafts / logq [gamma, bs] step-major; verify_tok / verify_logp / verify_logz [bs, G]: columns 0..gamma-1 hold
// log p_target of the drafts, column gamma the sampled bonus token and its logZ.
__global__ void write_back_kernel(SlotArrays a, const int* __restrict__ active, int bs, int gamma,
                                  const int* __restrict__ drafts, const float* __restrict__ logq,
                                  const int* __restrict__ verify_tok, const float* __restrict__ verify_logp,
                                  const float* __restrict__ verify_logz, float alpha, int use_logz,
                                  int* __restrict__ tokens_out, float* __restrict__ diff_out) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= bs) return;
  const int G = gamma + 1;
  const int slot = active[b];
  const int count = a.token_counts[slot];
  const bool was_finished = a.finished[slot] != 0;
  const bool ign = a.ignore_eos[slot] != 0;
  const int max_new = a.max_new_tokens[slot];
  int eos[MAX_EOS];
#pragma unroll
  for (int i = 0; i < MAX_EOS; ++i) eos[i] = a.eos_ids[slot * MAX_EOS + i];
  int first_eos = G;
  int matched = -1;
  for (int k = 0; k < G; ++k) {
    const int tok = k < gamma ? drafts[k * bs + b] : verify_tok[b * G + gamma];
    if (tokens_out) tokens_out[b * G + k] = tok;
    if (count + k < a.max_out) a.all_token_ids[(size_t)slot * a.max_out + count + k] = tok;
    if (!ign && first_eos == G) {
#pragma unroll
      for (int i = 0; i < MAX_EOS; ++i)
        if (eos[i] >= 0 && eos[i] == tok) { first_eos = k; matched = tok; }
    }
  }
  const int new_count = count + G;
  a.token_counts[slot] = new_count;
  a.verified_ids[slot] = verify_tok[b * G + gamma];
  a.prev_ids[slot] = drafts[(gamma - 1) * bs + b];
  const bool length_hit = new_count >= max_new;
  const bool eos_hit = first_eos < G;
  const bool newly = !was_finished && (length_hit || eos_hit);
  if (newly) {
    a.finished[slot] = 1;
    a.finish_code[slot] = length_hit ? 1 : 2;
    a.finished_len[slot] = length_hit ? max_new : count + first_eos + 1;
    a.matched_eos[slot] = (eos_hit && !length_hit) ? matched : -1;
  }
  int cutoff = gamma - 1;
  const bool eos_new = newly && eos_hit;
  if (eos_new && first_eos < cutoff) cutoff = first_eos;
  if (was_finished) cutoff = -1;
  double inc = 0.0;
  for (int k = 0; k < gamma; ++k) {
    const float d = alpha * verify_logp[b * G + k] - logq[k * bs + b];
    if (diff_out) diff_out[b * gamma + k] = d;
    if (k <= cutoff) inc += (double)d;
  }
  if (use_logz) {
    const bool eos_in_draft = eos_new && first_eos < gamma;
    if (!was_finished && !eos_in_draft) inc += (double)verify_logz[b * G + gamma];
  }
  a.log_weights[slot] += inc;
  a.interval_weights[slot] += inc;
}

// One warp per active group row; N <= 32.
__global__ void collect_kernel(SlotArrays a, const int* __restrict__ active_rows, int n_groups,
                               const int* __restrict__ group_to_slots, int N, double threshold,
                               unsigned long long seed, long long* __restrict__ counters,
                               double* __restrict__ group_log_z, int* __restrict__ job_dst,
                               int* __restrict__ job_src) {
  const int gi = blockIdx.x;
  if (gi >= n_groups) return;
  const int lane = threadIdx.x;
  const int row = active_rows[gi];
  const int slot = lane < N ? group_to_slots[row * N + lane] : -1;
  const double iw = slot >= 0 ? a.interval_weights[slot] : -INFINITY;
  double mx = iw;
  for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const double ex = slot >= 0 ? exp(iw - mx) : 0.0;
  double sum = ex, sq = ex * ex;
  for (int o = 16; o > 0; o >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
  }
  const double ess = (sum * sum) / sq;
  const bool go = N >= 2 && threshold > 0.0 && ess < threshold * (double)N;
  if (!go) return;
  // inclusive prefix sum of normalised weights
  const double w = ex / sum;
  double cdf = w;
  for (int o = 1; o < 32; o <<= 1) {
    const double t = __shfl_up_sync(0xffffffffu, cdf, o);
    if (lane >= o) cdf += t;
  }
  const double total = __shfl_sync(0xffffffffu, cdf, N - 1);
  cdf /= total;
  const Philox rng(seed);
  uint32_t rnd[4];
  const unsigned long long step = (unsigned long long)counters[0];
  rng.run((uint32_t)step, (uint32_t)(step >> 32), (uint32_t)row, 0u, rnd);
  const double u = u32_to_unit_d(rnd[0]);
  // ancestor of offspring `lane`
  const double pos = (u + (double)lane) / (double)N;
  int anc = 0;
  for (int j = 0; j < N; ++j) {
    const double cj = __shfl_sync(0xffffffffu, cdf, j);
    if (lane < N && cj < pos) anc += 1;
  }
  if (anc > N - 1) anc = N - 1;
  __shared__ int counts[32];
  counts[lane] = 0;
  __syncwarp();
  if (lane < N) atomicAdd(&counts[anc], 1);
  __syncwarp();
  if (lane == 0) {
    // dead particles in index order receive the surplus copies in index order (deterministic)
    int dead[32], nd = 0;
    for (int i = 0; i < N; ++i)
      if (counts[i] == 0) dead[nd++] = i;
    if (nd > 0) {
      const int base = (int)atomicAdd((unsigned long long*)&counters[1], (unsigned long long)nd);
      int k = 0;
      for (int i = 0; i < N && k < nd; ++i)
        for (int c = 1; c < counts[i] && k < nd; ++c) {
          job_dst[base + k] = group_to_slots[row * N + dead[k]];
          job_src[base + k] = group_to_slots[row * N + i];
          ++k;
        }
    }
    group_log_z[row] += mx + log(sum) - log((double)N);
    atomicAdd((unsigned long long*)&counters[2], 1ull);
  }
  if (slot >= 0) {
    a.interval_weights[slot] = 0.0;
    a.log_weights[slot] = 0.0;
  }
}

__global__ void __launch_bounds__(128)
resample_apply_kernel(SlotArrays a, const long long* __restrict__ counters, const int* __restrict__ job_dst,
                      const int* __restrict__ job_src) {
  const int job = blockIdx.x;
  if (job >= (int)counters[1]) return;
  const int dst = job_dst[job], src = job_src[job];
  int* bt_dst = a.block_table + (size_t)dst * a.bt_stride;
  const int* bt_src = a.block_table + (size_t)src * a.bt_stride;
  const int Ld = a.seq_lens[dst], Ls = a.seq_lens[src];
  // 1. release the destination's pages
  for (int j = threadIdx.x; j < Ld; j += blockDim.x) {
    const int page = bt_dst[j];
    if (page <= 0 || page > a.n_pages) continue;
    const int old = atomicSub(&a.refcount[page], 1);
    if (old == 1) {
      const int pos = atomicAdd(a.free_count, 1);
      a.free_stack[pos] = page;
    }
  }
  __syncthreads();
  // 2. share the ancestor's pages
  for (int j = threadIdx.x; j < Ls; j += blockDim.x) {
    const int page = bt_src[j];
    bt_dst[j] = page;
    if (page > 0 && page <= a.n_pages) atomicAdd(&a.refcount[page], 1);
  }
  // 3. lineage scalars and token history
  const int n_tok = a.token_counts[src];
  for (int j = threadIdx.x; j < n_tok && j < a.max_out; j += blockDim.x)
    a.all_token_ids[(size_t)dst * a.max_out + j] = a.all_token_ids[(size_t)src * a.max_out + j];
  if (threadIdx.x == 0) {
    a.seq_lens[dst] = Ls;
    a.verified_ids[dst] = a.verified_ids[src];
    a.prev_ids[dst] = a.prev_ids[src];
    a.token_counts[dst] = n_tok;
    a.finished[dst] = a.finished[src];
    a.finished_len[dst] = a.finished_len[src];
    a.finish_code[dst] = a.finish_code[src];
    a.matched_eos[dst] = a.matched_eos[src];
  }
}

// state [layers, rows, row_elems] (any 4-byte-multiple row); grid (max_jobs, layers, chunks)
__global__ void state_copy_kernel(uint8_t* __restrict__ state, long long layer_stride_bytes, long long row_bytes,
                                  const long long* __restrict__ counters, const int* __restrict__ job_dst,
                                  const int* __restrict__ job_src, int n_rows) {
  const int job = blockIdx.x;
  if (job >= (int)counters[1]) return;
  const int dst = job_dst[job], src = job_src[job];
  if (dst < 0 || src < 0 || dst >= n_rows || src >= n_rows) return;
  uint8_t* base = state + (size_t)blockIdx.y * layer_stride_bytes;
  const uint4* s = reinterpret_cast<const uint4*>(base + (size_t)src * row_bytes);
  uint4* d = reinterpret_cast<uint4*>(base + (size_t)dst * row_bytes);
  const long long nvec = row_bytes >> 4;
  for (long long i = (long long)blockIdx.z * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.z * blockDim.x)
    d[i] = s[i];
}

}  // namespace smc

using smc::SlotArrays;

SMC_API int smc_slot_arrays_size() { return (int)sizeof(SlotArrays); }

SMC_API int smc_cycle_io_size() { return (int)sizeof(smc::CycleIO); }

SMC_API int smc_prepare_cycle(const SlotArrays* a, const int* active, int bs, int G, long long* counters,
                              const smc::CycleIO* io, cudaStream_t st) {
  if (bs <= 0) return 0;
  smc::prepare_cycle_kernel<<<1, 256, 0, st>>>(*a, active, bs, G, counters, *io);
  return (int)cudaGetLastError();
}

SMC_API int smc_assemble_verify(const smc::CycleIO* io, const int* drafts, int bs, int gamma, cudaStream_t st) {
  if (bs <= 0) return 0;
  smc::assemble_verify_kernel<<<(bs * (gamma + 1) + 127) / 128, 128, 0, st>>>(*io, drafts, bs, gamma);
  return (int)cudaGetLastError();
}

SMC_API int smc_write_back(const SlotArrays* a, const int* active, int bs, int gamma, const int* drafts,
                           const float* logq, const int* verify_tok, const float* verify_logp,
                           const float* verify_logz, float alpha, int use_logz, int* tokens_out, float* diff_out,
                           cudaStream_t st) {
  if (bs <= 0) return 0;
  smc::write_back_kernel<<<(bs + 63) / 64, 64, 0, st>>>(*a, active, bs, gamma, drafts, logq, verify_tok, verify_logp,
                                                        verify_logz, alpha, use_logz, tokens_out, diff_out);
  return (int)cudaGetLastError();
}

SMC_API int smc_collect_resample(const SlotArrays* a, const int* active_rows, int n_groups, const int* group_to_slots,
                                 int N, double threshold, unsigned long long seed, long long* counters,
                                 double* group_log_z, int* job_dst, int* job_src, cudaStream_t st) {
  if (n_groups <= 0) return 0;
  if (N > 32) return -60;
  smc::collect_kernel<<<n_groups, 32, 0, st>>>(*a, active_rows, n_groups, group_to_slots, N, threshold, seed, counters,
                                               group_log_z, job_dst, job_src);
  if (N >= 2)
    smc::resample_apply_kernel<<<n_groups * (N - 1), 128, 0, st>>>(*a, counters, job_dst, job_src);
  return (int)cudaGetLastError();
}

// Applies a job list produced elsewhere (the particle-parallel collect kernel) to local ancestors.
SMC_API int smc_resample_apply(const SlotArrays* a, const long long* counters, const int* job_dst, const int* job_src,
                               int max_jobs, cudaStream_t st) {
  if (max_jobs <= 0) return 0;
  smc::resample_apply_kernel<<<max_jobs, 128, 0, st>>>(*a, counters, job_dst, job_src);
  return (int)cudaGetLastError();
}

SMC_API int smc_state_copy(void* state, long long layer_stride_bytes, long long row_bytes, int n_layers, int n_rows,
                           const long long* counters, const int* job_dst, const int* job_src, int max_jobs,
                           cudaStream_t st) {
  if (max_jobs <= 0 || n_layers <= 0) return 0;
  if (row_bytes & 15) return -61;
  int chunks = (int)((row_bytes / 16 + 255) / 256);
  if (chunks > 16) chunks = 16;
  smc::state_copy_kernel<<<dim3(max_jobs, n_layers, chunks), 256, 0, st>>>((uint8_t*)state, layer_stride_bytes, row_bytes,
                                                                        counters, job_dst, job_src, n_rows);
  return (int)cudaGetLastError();
}
