// Particle-parallel resampling: the N particles of a group are sharded over R ranks (N_local each),
// every rank holds full model replicas and its own paged KV / recurrent-state pools.  Each cycle
//   pp_share_weights  every rank stores its particles' interval log-weights into all ranks' gather
//                     buffers (peer stores) and bumps their counters
//   pp_collect        every rank waits (bounded) for all shards, runs the same ESS test and systematic
//                     resampling over the N global particles with the same Philox offset, and keeps
//                     the jobs whose destination it owns: local jobs (ancestor on this rank) and
//                     remote jobs (ancestor on another GPU)
//   pp_release / pp_adopt / pp_copy   for remote jobs: drop the destination's post-prompt pages, pop
//                     fresh local pages, rewrite the block table, copy lineage scalars and token
//                     history from the peer, then gather the ancestor's post-prompt KV rows of every
//                     layer of both models and its recurrent state over NVLink (plain peer loads).
//                     The prompt prefix is replicated per rank, so only suffix pages ever cross GPUs.
//   pp_barrier        all ranks check in before the next cycle mutates state that peers were reading
#include "common.cuh"

namespace smc {

constexpr int PP_MAX_RANKS = 8;
constexpr int PP_MAX_TENSORS = 8;

struct PpTensor {            // [layers, rows, row_bytes]
  unsigned long long base;   // device address on the owning rank (peer-mapped)
  long long layer_stride;    // bytes
  long long row_bytes;
  int n_layers;
  int by_slot;               // 1: rows are indexed by slot (recurrent state), 0: by page id (KV)
};

struct PpRank {
  const int* seq_lens;
  const int* verified_ids;
  const int* prev_ids;
  const int* token_counts;
  const uint8_t* finished;
  const int* finished_len;
  const int* finish_code;
  const int* matched_eos;
  const int* all_token_ids;
  const int* block_table;
  const int* group_to_slots;
  PpTensor t[PP_MAX_TENSORS];
};

struct PpWorld {
  PpRank r[PP_MAX_RANKS];
  unsigned long long heap_base[PP_MAX_RANKS];
  int n_ranks, rank, n_tensors, n_local;      // n_local particles per group per rank
  int max_out, bt_stride, max_groups, pad;
};

struct PpLocal {              // this rank's mutable arrays
  int* seq_lens; int* verified_ids; int* prev_ids; int* token_counts; uint8_t* finished; int* finished_len;
  int* finish_code; int* matched_eos; int* all_token_ids; int* block_table; const int* prompt_lens;
  double* log_weights; double* interval_weights;
  int* refcount; int* free_stack; int* free_count; int* alloc_error; int n_pages;
};

// ---- 1. share weights --------------------------------------------------------------------------
// gather buffer on every rank: double [n_ranks, max_groups, n_local + 1]; the extra entry of a row carries
// the number of this rank's particles of the group that are still unfinished
__global__ void pp_share_weights_kernel(const PpWorld* __restrict__ w, const double* __restrict__ interval,
                                        const uint8_t* __restrict__ finished, const int* __restrict__ active_rows,
                                        int n_groups, const int* __restrict__ group_to_slots, long long gather_off,
                                        long long flag_off) {
  const PpWorld& W = *w;
  const int stride = W.n_local + 1;
  const int total = n_groups * stride;
  for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const int gi = idx / stride, i = idx % stride;
    const int row = active_rows[gi];
    double v;
    if (i < W.n_local) {
      v = interval[group_to_slots[row * W.n_local + i]];
    } else {
      int alive = 0;
      for (int k = 0; k < W.n_local; ++k) alive += finished[group_to_slots[row * W.n_local + k]] ? 0 : 1;
      v = (double)alive;
    }
    for (int pr = 0; pr < W.n_ranks; ++pr) {
      double* dst = reinterpret_cast<double*>(W.heap_base[pr] + gather_off) +
                    ((size_t)W.rank * W.max_groups + row) * stride + i;
      *dst = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < W.n_ranks)
    atomicAdd_system(reinterpret_cast<unsigned long long*>(W.heap_base[threadIdx.x] + flag_off), 1ull);
}

// ---- 2. collect -----------------------------------------------------------------------------------
// counters: [0] cycle step, [1] local jobs, [2] groups resampled, [3] remote jobs
__global__ void pp_collect_kernel(const PpWorld* __restrict__ w, PpLocal loc, const double* __restrict__ gather,
                                  const unsigned long long* __restrict__ flag, const int* __restrict__ active_rows,
                                  int n_groups, const int* __restrict__ group_to_slots, double threshold,
                                  unsigned long long seed, long long* __restrict__ counters,
                                  double* __restrict__ group_log_z, int* __restrict__ job_dst,
                                  int* __restrict__ job_src, int* __restrict__ rjob_dst, int* __restrict__ rjob_rank,
                                  int* __restrict__ rjob_idx, int* __restrict__ group_active, int* status) {
  const PpWorld& W = *w;
  const int gi = blockIdx.x, lane = threadIdx.x;
  if (gi >= n_groups) return;
  __shared__ int ok;
  if (lane == 0) {
    ok = wait_counter_sys(flag, (unsigned long long)counters[0] * (unsigned long long)W.n_ranks) ? 1 : 0;
    if (!ok) atomicOr(status, SMC_ERR_PEER_TIMEOUT);
  }
  __syncwarp();
  // A shard that never arrived leaves stale weights in the gather buffer; a plan made from them would differ from
  // the peers' plans and could name an ancestor whose rank has not populated it.  Such a rank resamples nothing this
  // cycle (no local jobs, no peer reads); the status word tells the host.
  if (!ok) return;
  const int N = W.n_ranks * W.n_local;
  const int row = active_rows[gi];
  const int pr = lane / W.n_local, pi = lane % W.n_local;       // global particle `lane` lives on rank pr
  const bool have = lane < N;
  const int stride = W.n_local + 1;
  const double iw = have ? gather[((size_t)pr * W.max_groups + row) * stride + pi] : -INFINITY;
  {  // particles of this group that are still running, over all ranks (same value on every rank)
    double alive = lane < W.n_ranks ? gather[((size_t)lane * W.max_groups + row) * stride + W.n_local] : 0.0;
    for (int o = 16; o > 0; o >>= 1) alive += __shfl_xor_sync(0xffffffffu, alive, o);
    if (lane == 0) group_active[row] = (int)(alive + 0.5);
  }
  double mx = iw;
  for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const double ex = have ? exp(iw - mx) : 0.0;
  double sum = ex, sq = ex * ex;
  for (int o = 16; o > 0; o >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
  }
  const double ess = (sum * sum) / sq;
  const bool go = N >= 2 && threshold > 0.0 && ess < threshold * (double)N;
  if (!go) return;
  double cdf = ex / sum;
  for (int o = 1; o < 32; o <<= 1) {
    const double t = __shfl_up_sync(0xffffffffu, cdf, o);
    if (lane >= o) cdf += t;
  }
  cdf /= __shfl_sync(0xffffffffu, cdf, N - 1);
  const Philox rng(seed);
  uint32_t rnd[4];
  const unsigned long long step = (unsigned long long)counters[0];
  rng.run((uint32_t)step, (uint32_t)(step >> 32), (uint32_t)row, 0u, rnd);
  const double u = u32_to_unit_d(rnd[0]);
  const double pos = (u + (double)lane) / (double)N;
  int anc = 0;
  for (int j = 0; j < N; ++j) {
    const double cj = __shfl_sync(0xffffffffu, cdf, j);
    if (have && cj < pos) anc += 1;
  }
  if (anc > N - 1) anc = N - 1;
  __shared__ int counts[32];
  counts[lane] = 0;
  __syncwarp();
  if (have) atomicAdd(&counts[anc], 1);
  __syncwarp();
  if (lane == 0) {
    int dead[32], nd = 0;
    for (int i = 0; i < N; ++i)
      if (counts[i] == 0) dead[nd++] = i;
    int k = 0;
    for (int i = 0; i < N && k < nd; ++i)
      for (int c = 1; c < counts[i] && k < nd; ++c, ++k) {
        const int d = dead[k];
        if (d / W.n_local != W.rank) continue;                 // another rank owns this destination
        const int dslot = group_to_slots[row * W.n_local + d % W.n_local];
        if (i / W.n_local == W.rank) {
          const int at = (int)atomicAdd((unsigned long long*)&counters[1], 1ull);
          job_dst[at] = dslot;
          job_src[at] = group_to_slots[row * W.n_local + i % W.n_local];
        } else {
          const int at = (int)atomicAdd((unsigned long long*)&counters[3], 1ull);
          rjob_dst[at] = dslot;
          rjob_rank[at] = i / W.n_local;
          rjob_idx[at] = row * W.n_local + i % W.n_local;     // index into the peer's group_to_slots
        }
      }
    group_log_z[row] += mx + log(sum) - log((double)N);
    atomicAdd((unsigned long long*)&counters[2], 1ull);
  }
  // every local particle of a resampled group restarts with zero weight
  if (lane < W.n_local) {
    const int slot = group_to_slots[row * W.n_local + lane];
    loc.interval_weights[slot] = 0.0;
    loc.log_weights[slot] = 0.0;
  }
}

// ---- 3. remote jobs ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
pp_release_kernel(PpLocal loc, int bt_stride, const long long* __restrict__ counters, const int* __restrict__ rjob_dst) {
  const int job = blockIdx.x;
  if (job >= (int)counters[3]) return;
  const int dst = rjob_dst[job];
  int* bt = loc.block_table + (size_t)dst * bt_stride;
  const int L = loc.seq_lens[dst], P = loc.prompt_lens[dst];
  for (int j = P + threadIdx.x; j < L; j += blockDim.x) {
    const int page = bt[j];
    if (page <= 0 || page > loc.n_pages) continue;
    if (atomicSub(&loc.refcount[page], 1) == 1) loc.free_stack[atomicAdd(loc.free_count, 1)] = page;
  }
}

__global__ void __launch_bounds__(128)
pp_adopt_kernel(const PpWorld* __restrict__ w, PpLocal loc, const long long* __restrict__ counters,
                const int* __restrict__ rjob_dst, const int* __restrict__ rjob_rank, const int* __restrict__ rjob_idx,
                int* __restrict__ rjob_src_slot, int* status) {
  const PpWorld& W = *w;
  const int job = blockIdx.x;
  if (job >= (int)counters[3]) return;
  __shared__ int s_base, s_src, s_len;
  const int dst = rjob_dst[job];
  const PpRank& peer = W.r[rjob_rank[job]];
  const int P = loc.prompt_lens[dst];
  if (threadIdx.x == 0) {
    // everything read from the peer is checked before it becomes an index: a slot or a length outside its range
    // (a peer that has not set the group up) ends the job here, with the destination left as it is
    int src = peer.group_to_slots[rjob_idx[job]];
    int Lp = -1;
    if (src >= 0 && src < W.max_groups * W.n_local) Lp = peer.seq_lens[src];
    if (Lp < P || Lp > W.bt_stride) {
      atomicOr(status, SMC_ERR_BOUNDS);
      src = -1;
      s_base = -1;
    } else {
      const int n_new = Lp - P;
      const int old = atomicSub(loc.free_count, n_new);
      if (old < n_new) {                     // pool ran dry: fall back to the scratch page and report
        atomicAdd(loc.free_count, n_new);
        atomicOr(loc.alloc_error, SMC_ERR_ALLOC_EXHAUSTED);
        s_base = -1;
      } else {
        s_base = old - n_new;
      }
    }
    s_src = src;
    s_len = Lp;
    rjob_src_slot[job] = src;
  }
  __syncthreads();
  const int src = s_src, base = s_base;
  if (src < 0) return;
  const int Ls = s_len;
  int* bt = loc.block_table + (size_t)dst * W.bt_stride;
  for (int j = P + threadIdx.x; j < Ls; j += blockDim.x) {
    int page = 0;
    if (base >= 0) {
      page = loc.free_stack[base + (j - P)];
      loc.refcount[page] = 1;
    }
    bt[j] = page;
  }
  const int n_tok = peer.token_counts[src];
  for (int j = threadIdx.x; j < n_tok && j < W.max_out; j += blockDim.x)
    loc.all_token_ids[(size_t)dst * W.max_out + j] = peer.all_token_ids[(size_t)src * W.max_out + j];
  if (threadIdx.x == 0) {
    loc.seq_lens[dst] = Ls;
    loc.verified_ids[dst] = peer.verified_ids[src];
    loc.prev_ids[dst] = peer.prev_ids[src];
    loc.token_counts[dst] = n_tok;
    loc.finished[dst] = peer.finished[src];
    loc.finished_len[dst] = peer.finished_len[src];
    loc.finish_code[dst] = peer.finish_code[src];
    loc.matched_eos[dst] = peer.matched_eos[src];
  }
}

// grid (max remote jobs, total layers over all tensors, token chunks)
__global__ void __launch_bounds__(256)
pp_copy_kernel(const PpWorld* __restrict__ w, PpLocal loc, const long long* __restrict__ counters,
               const int* __restrict__ rjob_dst, const int* __restrict__ rjob_rank,
               const int* __restrict__ rjob_src_slot) {
  const PpWorld& W = *w;
  const int job = blockIdx.x;
  if (job >= (int)counters[3]) return;
  int lay = blockIdx.y, ti = 0;
  while (ti < W.n_tensors && lay >= W.r[W.rank].t[ti].n_layers) { lay -= W.r[W.rank].t[ti].n_layers; ++ti; }
  if (ti >= W.n_tensors) return;
  const int dst = rjob_dst[job], src = rjob_src_slot[job], pr = rjob_rank[job];
  if (src < 0) return;                         // adopt refused this job
  const PpTensor& ts = W.r[pr].t[ti];
  const PpTensor& td = W.r[W.rank].t[ti];
  const long long rb = td.row_bytes;
  const uint4* sbase = reinterpret_cast<const uint4*>(ts.base + (unsigned long long)lay * ts.layer_stride);
  uint4* dbase = reinterpret_cast<uint4*>(td.base + (unsigned long long)lay * td.layer_stride);
  const long long vec = rb >> 4;
  if (td.by_slot) {            // recurrent state: one row per slot
    const uint4* s = sbase + (size_t)src * vec;
    uint4* d = dbase + (size_t)dst * vec;
    for (long long i = (long long)blockIdx.z * blockDim.x + threadIdx.x; i < vec; i += (long long)gridDim.z * blockDim.x)
      d[i] = s[i];
    return;
  }
  const int P = loc.prompt_lens[dst], Ls = loc.seq_lens[dst];     // adopt already set the new length
  const int* bt_src = W.r[pr].block_table + (size_t)src * W.bt_stride;
  const int* bt_dst = loc.block_table + (size_t)dst * W.bt_stride;
  const int lanes_per_row = (int)(vec < 32 ? vec : 32);
  const int rows_per_block = blockDim.x / lanes_per_row;
  const int sub = threadIdx.x / lanes_per_row, l = threadIdx.x % lanes_per_row;
  for (int j = P + blockIdx.z * rows_per_block + sub; j < Ls; j += gridDim.z * rows_per_block) {
    const int ps = bt_src[j], pd = bt_dst[j];
    if (pd <= 0 || ps < 0 || ps > loc.n_pages) continue;
    const uint4* s = sbase + (size_t)ps * vec;
    uint4* d = dbase + (size_t)pd * vec;
    for (long long i = l; i < vec; i += lanes_per_row) d[i] = s[i];
  }
}

// ---- 4. barrier --------------------------------------------------------------------------------------
__global__ void pp_barrier_kernel(const PpWorld* __restrict__ w, long long flag_off,
                                  const unsigned long long* __restrict__ flag_local,
                                  const long long* __restrict__ counters, int* status, int phase) {
  const PpWorld& W = *w;
  __threadfence_system();
  if (phase != 2 && (int)threadIdx.x < W.n_ranks)
    atomicAdd_system(reinterpret_cast<unsigned long long*>(W.heap_base[threadIdx.x] + flag_off), 1ull);
  if (phase != 1 && threadIdx.x == 0) {
    if (!wait_counter_sys(flag_local, (unsigned long long)counters[0] * (unsigned long long)W.n_ranks))
      atomicOr(status, SMC_ERR_PEER_TIMEOUT);
  }
}

}  // namespace smc

using namespace smc;

SMC_API int smc_pp_world_size() { return (int)sizeof(PpWorld); }
SMC_API int smc_pp_local_size() { return (int)sizeof(PpLocal); }

// phases let a single-GPU emulation interleave the ranks: 1 = share, 2 = collect + local/remote apply, 3 = barrier
SMC_API int smc_pp_share_weights(const PpWorld* w_dev, const double* interval, const uint8_t* finished,
                                 const int* active_rows, int n_groups, const int* group_to_slots, long long gather_off, long long flag_off, cudaStream_t st) {
  if (n_groups <= 0) return 0;
  pp_share_weights_kernel<<<1, 256, 0, st>>>(w_dev, interval, finished, active_rows, n_groups, group_to_slots, gather_off,
                                             flag_off);
  return (int)cudaGetLastError();
}

SMC_API int smc_pp_collect(const PpWorld* w_dev, const PpLocal* loc, const double* gather,
                           const unsigned long long* flag, const int* active_rows, int n_groups,
                           const int* group_to_slots, double threshold, unsigned long long seed, long long* counters,
                           double* group_log_z, int* job_dst, int* job_src, int* rjob_dst, int* rjob_rank,
                           int* rjob_idx, int* group_active, int* status, cudaStream_t st) {
  if (n_groups <= 0) return 0;
  pp_collect_kernel<<<n_groups, 32, 0, st>>>(w_dev, *loc, gather, flag, active_rows, n_groups, group_to_slots,
                                             threshold, seed, counters, group_log_z, job_dst, job_src, rjob_dst,
                                             rjob_rank, rjob_idx, group_active, status);
  return (int)cudaGetLastError();
}

SMC_API int smc_pp_fetch(const PpWorld* w_dev, const PpLocal* loc, int bt_stride, const long long* counters,
                         const int* rjob_dst, const int* rjob_rank, const int* rjob_idx, int* rjob_src_slot,
                         int max_jobs, int total_layers, int phase, int* status, cudaStream_t st) {
  if (max_jobs <= 0) return 0;
  if (phase == 0 || phase == 1)
    pp_release_kernel<<<max_jobs, 128, 0, st>>>(*loc, bt_stride, counters, rjob_dst);
  if (phase == 0 || phase == 2) {
    pp_adopt_kernel<<<max_jobs, 128, 0, st>>>(w_dev, *loc, counters, rjob_dst, rjob_rank, rjob_idx, rjob_src_slot,
                                              status);
    if (total_layers > 0)
      pp_copy_kernel<<<dim3(max_jobs, total_layers, 8), 256, 0, st>>>(w_dev, *loc, counters, rjob_dst, rjob_rank,
                                                                     rjob_src_slot);
  }
  return (int)cudaGetLastError();
}

SMC_API int smc_pp_barrier(const PpWorld* w_dev, long long flag_off, const unsigned long long* flag_local,
                           const long long* counters, int* status, int phase, cudaStream_t st) {
  // phase 0: check in and wait; 1: check in only; 2: wait only (single-GPU emulation of several ranks)
  pp_barrier_kernel<<<1, 32, 0, st>>>(w_dev, flag_off, flag_local, counters, status, phase);
  return (int)cudaGetLastError();
}
