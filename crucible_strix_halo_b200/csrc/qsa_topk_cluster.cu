// Exact top-512 of a long score row with a thread-block CLUSTER of 8 CTAs per row (sm_100a).
//
// Same total order and output as the single-CTA select in qsa_select.cu (score desc, block id asc, ascending
// emit; LaunchQsaTop, engine/layers/qsa_long.h:111-380), for rows with more than 8192 blocks.  Each CTA keeps
// its contiguous eighth of the row in registers; every radix pass builds a local 256-bin histogram in shared
// memory, the eight histograms are summed through distributed shared memory, and every CTA takes the same
// decision.  The emit offsets of a CTA are the totals of the CTAs before it, read the same way.  Eight SMs read
// the row in parallel and no pass re-reads it.
#include <cooperative_groups.h>
#include "qsa.cuh"

namespace cg = cooperative_groups;

namespace cr {

// kClusterCtas CTAs per row: 8 for the few rows of a decode / verify step (shortest latency per row), 2 for the
// many rows of a prefill part (each CTA then holds 32 values per thread and more rows run at once).
template <int kClusterCtas, int PT>
__global__ void __cluster_dims__(kClusterCtas, 1, 1) __launch_bounds__(1024) qsa_topk_cluster_kernel(const __grid_constant__ QsaParams P) {
  pdl_release();
  pdl_wait();
  const cr_qsa_args& a = P.span[blockIdx.y];
  const int r = blockIdx.x / kClusterCtas;
  if (r >= a.R) return;                                   // uniform over the cluster
  const int nb = (a.pos0 + r + 1) / 4;
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  if (nb <= CR_SEL_BLOCKS) { if (rank == 0 && t == 0) a.nsel[r] = -1; return; }

  __shared__ unsigned hist[8][256];
  __shared__ unsigned histsum[256];        // read by the whole cluster
  __shared__ unsigned totals[2];           // this CTA's (gt, eq), read by the higher ranks
  __shared__ unsigned wtot[32], gt_pre[33], eq_pre[33];
  __shared__ unsigned s_prefix, s_remaining;

  const int chunk = ((nb + kClusterCtas - 1) / kClusterCtas + 31) & ~31;   // ids per CTA, multiple of 32
  const int cbase = rank * chunk, cend = min(cbase + chunk, nb);
  const int per = (chunk + 1023) / 1024;                                    // <= PT by the launcher
  const int span = per * 32, begin = cbase + w * span, end = min(begin + span, cend);
  const float* sc = a.scores + (size_t)r * a.sstride;
  unsigned u[PT];
  unsigned vmask = 0u;
#pragma unroll
  for (int i = 0; i < PT; ++i) {
    const int idx = begin + 32 * i + l;
    const bool valid = i < per && idx < end;
    u[i] = valid ? __float_as_uint(sc[idx]) : 0u;
    if (valid) vmask |= 1u << i;
  }
  if (t == 0) { s_prefix = 0u; s_remaining = CR_SEL_BLOCKS; }
  unsigned mask = 0u;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = t; i < 8 * 256; i += 1024) (&hist[0][0])[i] = 0u;
    __syncthreads();
    const unsigned prefix = s_prefix, remaining = s_remaining;
    unsigned last = 0u, run = 0u;
#pragma unroll
    for (int i = 0; i < PT; ++i) {
      if (!((vmask >> i) & 1u) || (u[i] & mask) != prefix) continue;
      const unsigned bin = (u[i] >> shift) & 255u;
      if (run && bin != last) { atomicAdd(&hist[w & 7][last], run); run = 0u; }
      last = bin; ++run;
    }
    if (run) atomicAdd(&hist[w & 7][last], run);
    __syncthreads();
    if (t < 256) {
      unsigned c = 0u;
#pragma unroll
      for (int rep = 0; rep < 8; ++rep) c += hist[rep][t];
      histsum[t] = c;
    }
    cluster.sync();                                        // every CTA's histsum is complete
    unsigned c = 0u, inc = 0u;
    if (t < 256) {                                         // thread j looks at bin 255 - j (descending keys)
#pragma unroll
      for (int k = 0; k < kClusterCtas; ++k) c += cluster.map_shared_rank(histsum, k)[255 - t];
      inc = c;
#pragma unroll
      for (int step = 1; step < 32; step <<= 1) {
        const unsigned v = __shfl_up_sync(0xffffffffu, inc, step);
        if (l >= step) inc += v;
      }
      if (l == 31) wtot[w] = inc;
    }
    __syncthreads();
    if (t < 256) {
      for (int ww = 0; ww < w; ++ww) inc += wtot[ww];
      const unsigned exc = inc - c;
      if (exc < remaining && inc >= remaining) {
        s_prefix = prefix | ((unsigned)(255 - t) << shift);
        s_remaining = remaining - exc;
      }
    }
    cluster.sync();                                        // remote reads of histsum done; decision visible
    mask |= 255u << shift;
  }
  const unsigned thr = s_prefix, need = s_remaining;
  unsigned gt = 0u, eq = 0u;
#pragma unroll
  for (int i = 0; i < PT; ++i)
    if ((vmask >> i) & 1u) { gt += u[i] > thr; eq += u[i] == thr; }
#pragma unroll
  for (int step = 16; step > 0; step >>= 1) {
    gt += __shfl_xor_sync(0xffffffffu, gt, step);
    eq += __shfl_xor_sync(0xffffffffu, eq, step);
  }
  if (l == 0) { gt_pre[w + 1] = gt; eq_pre[w + 1] = eq; }
  __syncthreads();
  if (t == 0) {
    gt_pre[0] = eq_pre[0] = 0u;
    for (int ww = 1; ww <= 32; ++ww) { gt_pre[ww] += gt_pre[ww - 1]; eq_pre[ww] += eq_pre[ww - 1]; }
    totals[0] = gt_pre[32]; totals[1] = eq_pre[32];
  }
  cluster.sync();                                          // totals of every CTA visible (also a block barrier)
  unsigned gt_before = 0u, eq_before = 0u;
  for (int k = 0; k < rank; ++k) {
    const unsigned* tk = cluster.map_shared_rank(totals, k);
    gt_before += tk[0]; eq_before += tk[1];
  }
  unsigned tie = eq_before + eq_pre[w];
  unsigned out = gt_before + gt_pre[w] + min(tie, need);
  const unsigned lower = (1u << l) - 1u;
  int* selected = a.sel + (size_t)r * CR_SEL_BLOCKS;
#pragma unroll
  for (int i = 0; i < PT; ++i) {
    if (begin + 32 * i >= end) break;                      // warp uniform
    const bool valid = (vmask >> i) & 1u;
    const unsigned eqmask = __ballot_sync(0xffffffffu, valid && u[i] == thr);
    const bool keep = valid && (u[i] > thr || (u[i] == thr && tie + __popc(eqmask & lower) < need));
    const unsigned chosen = __ballot_sync(0xffffffffu, keep);
    if (keep) selected[out + __popc(chosen & lower)] = begin + 32 * i + l;
    tie += __popc(eqmask);
    out += __popc(chosen);
  }
  if (rank == 0 && t == 0) a.nsel[r] = CR_SEL_BLOCKS;
  cluster.sync();                                          // no CTA exits while its totals may still be read
}

// nb_max in (8192, 262144]: PT = ceil(ceil(nb / ctas) / 1024) rounded to 8 / 16 / 32.
template <int CTAS>
static cr_status topk_cluster_launch_t(const QsaParams& P, int Rmax, int n, int nb_max, cudaStream_t stream) {
  const dim3 grid(CTAS * Rmax, n);
  const int per = (((nb_max + CTAS - 1) / CTAS + 31) / 32 * 32 + 1023) / 1024;
  if (per <= 8) CR_CUDA(launch_pdl(qsa_topk_cluster_kernel<CTAS, 8>, grid, dim3(1024), 0, stream, P));
  else if (per <= 16) CR_CUDA(launch_pdl(qsa_topk_cluster_kernel<CTAS, 16>, grid, dim3(1024), 0, stream, P));
  else if (per <= 32) CR_CUDA(launch_pdl(qsa_topk_cluster_kernel<CTAS, 32>, grid, dim3(1024), 0, stream, P));
  else { set_error("qsa top-k: %d blocks exceed the cluster select's range", nb_max); return CR_ERR_UNSUPPORTED; }
  CR_LAUNCH_CHECK("qsa_topk_cluster_kernel");
  return CR_OK;
}

cr_status qsa_topk_cluster_launch(const QsaParams& P, int Rmax, int n, int nb_max, cudaStream_t stream) {
  const bool many_rows = (long long)Rmax * n > 64 && nb_max <= 2 * 32 * 1024;
  return many_rows ? topk_cluster_launch_t<2>(P, Rmax, n, nb_max, stream) : topk_cluster_launch_t<8>(P, Rmax, n, nb_max, stream);
}

}  // namespace cr
