// Mixture-of-experts routing and data movement: fused router projection + softmax + top-k,
// deterministic (atomics-free) expert counts / offsets / tile table / slot assignment,
// dispatch of quantised rows into expert-contiguous slots, and the weighted combine.
// Replaces router_projection / router_topk (kernels/cuda/model/moe.py:16,413),
// expert_histogram* / expert_offsets / expert_tiles (moe.py:177-286,558-713),
// expert_dispatch (moe.py:286) and moe_combine (moe.py:498-557) of the reference.
#include "api.h"
#include "common.cuh"
#include "tp_comm.cuh"

namespace orinfer {

// ---------------------------------------------------------------- router + top-k
// One CTA per token row.  logits[e] = x[row] . W[e] (fp16 inputs, fp32 accumulate);
// softmax over the first `experts` rows of W; top-k by repeated argmax with ties going to
// the lower expert id; optional renormalisation; row `experts` of W (when present) is the
// shared-expert gate, returned as sigmoid(logit).
__global__ void __launch_bounds__(256) router_topk_kernel(
    const __half* __restrict__ x, const __half* __restrict__ w, int hidden, int experts,
    int has_shared, int top_k, int renorm, int* __restrict__ ids, float* __restrict__ probs,
    float* __restrict__ shared_gate) {
  extern __shared__ float logits[];                 // [experts + 1]
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nw = blockDim.x >> 5, total = experts + (has_shared ? 1 : 0);
  const __half* xr = x + static_cast<size_t>(row) * hidden;
  for (int e = warp; e < total; e += nw) {
    const __half* wr = w + static_cast<size_t>(e) * hidden;
    float acc = 0.f;
    for (int i = lane * 8; i < hidden; i += 256) {
      const int4 xa = *reinterpret_cast<const int4*>(xr + i);
      const int4 wa = *reinterpret_cast<const int4*>(wr + i);
      const __half2* xh = reinterpret_cast<const __half2*>(&xa);
      const __half2* wh = reinterpret_cast<const __half2*>(&wa);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = __half22float2(xh[j]), b = __half22float2(wh[j]);
        acc = fmaf(a.x, b.x, acc);
        acc = fmaf(a.y, b.y, acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) logits[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  // softmax statistics over the routed experts
  float mx = -INFINITY;
  for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, logits[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) sum += expf(logits[e] - mx);
  sum = warp_sum(sum);
  float chosen_sum = 0.f;
  for (int k = 0; k < top_k; ++k) {
    float best = -INFINITY;
    int bidx = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = logits[e];
      if (v > best) { best = v; bidx = e; }           // ascending e: first maximum wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
      if (ov > best || (ov == best && oi < bidx)) { best = ov; bidx = oi; }
    }
    const float p = expf(best - mx) / sum;
    if (lane == 0) {
      ids[row * top_k + k] = bidx;
      probs[row * top_k + k] = p;
      logits[bidx] = -INFINITY;
    }
    chosen_sum += p;
    __syncwarp();
  }
  if (renorm && lane == 0)
    for (int k = 0; k < top_k; ++k) probs[row * top_k + k] /= chosen_sum;
  if (has_shared && lane == 0)
    shared_gate[row] = 1.f / (1.f + expf(-logits[experts]));
}

// ---------------------------------------------------------------- counts (one CTA per expert)
// Under expert parallelism a rank owns experts [base, base + gridDim.x): ids outside that
// range are left to their owners (their slot stays -1 and the combine skips them).
__global__ void __launch_bounds__(256) moe_count_kernel(const int* __restrict__ ids, int assigns,
                                                        int base_expert,
                                                        int* __restrict__ counts) {
  const int e = blockIdx.x;
  int c = 0;
  for (int i = threadIdx.x; i < assigns; i += blockDim.x) c += ids[i] == e + base_expert;
  __shared__ int red[8];
  c = static_cast<int>(warp_sum(static_cast<float>(c)));       // counts < 2^24: exact
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int i = 0; i < 8; ++i) t += red[i];
    counts[e] = t;
  }
}

// offsets[e] = exclusive prefix of counts; tile table (expert, first slot, valid rows) for
// 128-row tiles; meta[0] = number of tiles.  One thread: E <= 512.
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int experts,
                                   int* __restrict__ offsets, int* __restrict__ tiles,
                                   int* __restrict__ meta, int max_tiles) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int off = 0, nt = 0;
  for (int e = 0; e < experts; ++e) {
    offsets[e] = off;
    const int c = counts[e];
    for (int r = 0; r < c && nt < max_tiles; r += 128) {
      tiles[nt * 4 + 0] = e;
      tiles[nt * 4 + 1] = off + r;
      tiles[nt * 4 + 2] = min(128, c - r);
      tiles[nt * 4 + 3] = 0;
      ++nt;
    }
    off += c;
  }
  offsets[experts] = off;
  meta[0] = nt;
}

// slot[i] = offsets[e] + rank of assignment i among the assignments of expert e (stable in
// (row, k) order); also copies the quantised row and its scale into that slot.
__global__ void __launch_bounds__(256) moe_dispatch_kernel(
    const int* __restrict__ ids, int assigns, int top_k, int base_expert,
    const int* __restrict__ offsets, const int8_t* __restrict__ q8,
    const float* __restrict__ scale, int K, int* __restrict__ slots,
    int8_t* __restrict__ q8_sorted, float* __restrict__ scale_sorted) {
  const int e = blockIdx.x;
  __shared__ int wsum[8];
  __shared__ int base;
  if (threadIdx.x == 0) base = offsets[e];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int start = 0; start < assigns; start += 256) {
    const int i = start + threadIdx.x;
    const bool mine = i < assigns && ids[i] == e + base_expert;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) wsum[warp] = __popc(ballot);
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    int block_total = 0;
    for (int w = 0; w < 8; ++w) block_total += wsum[w];
    if (mine) {
      const int slot = base + before + __popc(ballot & ((1u << lane) - 1u));
      slots[i] = slot;
      if (q8 != nullptr) {                  // nullptr: only the slot numbering is wanted
        const int row = i / top_k;
        scale_sorted[slot] = scale[row];
        const int4* src = reinterpret_cast<const int4*>(q8 + static_cast<size_t>(row) * K);
        int4* dst = reinterpret_cast<int4*>(q8_sorted + static_cast<size_t>(slot) * K);
        for (int c = 0; c < K / 16; ++c) dst[c] = src[c];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) base += block_total;
    __syncthreads();
  }
}

// out[row] = fp16( sum_k prob[row,k] * expert_out[slot(row,k)] + gate[row] * shared[row] )
__global__ void __launch_bounds__(256) moe_combine_kernel(
    const __half* __restrict__ expert_out, const int* __restrict__ slots,
    const float* __restrict__ probs, int top_k, const __half* __restrict__ shared_out,
    const float* __restrict__ shared_gate, __half* __restrict__ out, int hidden,
    const PeerOut peers) {
  const int row = blockIdx.x;
  for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < top_k; ++k) {
      const float p = probs[row * top_k + k];
      const int slot = slots[row * top_k + k];
      if (slot < 0) continue;                        // routed to an expert of another rank
      const int4 raw =
          *reinterpret_cast<const int4*>(expert_out + static_cast<size_t>(slot) * hidden + i);
      const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(p, __half2float(h[j]), acc[j]);
    }
    if (shared_out != nullptr) {
      const float g = shared_gate[row];
      const int4 raw =
          *reinterpret_cast<const int4*>(shared_out + static_cast<size_t>(row) * hidden + i);
      const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(g, __half2float(h[j]), acc[j]);
    }
    __align__(16) __half o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2half_rn(acc[j]);
    if (peers.tp == 0) {
      *reinterpret_cast<int4*>(out + static_cast<size_t>(row) * hidden + i) =
          *reinterpret_cast<const int4*>(o);
    } else {
      // expert-parallel combine: this rank's partial row goes straight into slot [rank] of
      // every rank's inbox; the consumer norm kernel sums the tp partials
      const size_t off = (static_cast<size_t>(peers.rank) * peers.rows_cap + row) * hidden + i;
      for (int d = 0; d < peers.tp; ++d)
        *reinterpret_cast<int4*>(peers.inbox[d] + off) = *reinterpret_cast<const int4*>(o);
    }
  }
  if (peers.tp != 0) peer_signal_done(peers, gridDim.x);
}

}  // namespace orinfer

using namespace orinfer;

extern "C" {

int orinfer_router_topk(const __half* x, const __half* w, int rows, int hidden, int experts,
                        int has_shared, int top_k, int renorm, int* ids, float* probs,
                        float* shared_gate, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden % 8 || top_k < 1 || top_k > experts || experts > 4096) return -1;
  router_topk_kernel<<<rows, 256, (experts + 1) * sizeof(float), stream>>>(
      x, w, hidden, experts, has_shared, top_k, renorm, ids, probs, shared_gate);
  return static_cast<int>(cudaGetLastError());
}

// counts [E], offsets [E+1], tiles int32 [max_tiles,4] = (expert, first slot, rows, 0),
// meta[0] = tile count, slots [rows*top_k]; q8_sorted / scale_sorted get the dispatched rows.
int orinfer_moe_dispatch(const int* ids, int rows, int top_k, int experts, const int8_t* q8,
                         const float* scale, int K, int* counts, int* offsets, int* tiles,
                         int* meta, int max_tiles, int* slots, int8_t* q8_sorted,
                         float* scale_sorted, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K % 16) return -1;
  const int assigns = rows * top_k;
  moe_count_kernel<<<experts, 256, 0, stream>>>(ids, assigns, 0, counts);
  moe_offsets_kernel<<<1, 32, 0, stream>>>(counts, experts, offsets, tiles, meta, max_tiles);
  moe_dispatch_kernel<<<experts, 256, 0, stream>>>(ids, assigns, top_k, 0, offsets, q8, scale, K,
                                                   slots, q8_sorted, scale_sorted);
  return static_cast<int>(cudaGetLastError());
}

// Expert-parallel dispatch: this rank owns experts [base_expert, base_expert + local_experts);
// only rows routed there are counted and copied, every other slot is -1.
int orinfer_moe_dispatch_ep(const int* ids, int rows, int top_k, int base_expert,
                            int local_experts, const int8_t* q8, const float* scale, int K,
                            int* counts, int* offsets, int* tiles, int* meta, int max_tiles,
                            int* slots, int8_t* q8_sorted, float* scale_sorted,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K % 16) return -1;
  const int assigns = rows * top_k;
  cudaMemsetAsync(slots, 0xFF, sizeof(int) * assigns, stream);
  moe_count_kernel<<<local_experts, 256, 0, stream>>>(ids, assigns, base_expert, counts);
  moe_offsets_kernel<<<1, 32, 0, stream>>>(counts, local_experts, offsets, tiles, meta,
                                           max_tiles);
  moe_dispatch_kernel<<<local_experts, 256, 0, stream>>>(ids, assigns, top_k, base_expert,
                                                         offsets, q8, scale, K, slots, q8_sorted,
                                                         scale_sorted);
  return static_cast<int>(cudaGetLastError());
}

// Combine whose result rows are pushed into every rank's inbox (slot [rank]) over NVLink and
// signalled, instead of being written locally: the all-reduce of the expert-parallel partial
// sums is completed by the consumer norm kernel.
int orinfer_moe_combine_peer(const __half* expert_out, const int* slots, const float* probs,
                             int rows, int top_k, const __half* shared_out,
                             const float* shared_gate, const OrinferPeerOut* peers, int hidden,
                             cudaStream_t stream) {
  if (rows <= 0 || peers == nullptr) return -1;
  if (hidden % 8 || rows > peers->rows_cap) return -1;
  if (peers->tp < 1 || peers->tp > TP_MAX) return -1;
  PeerOut po;
  for (int i = 0; i < TP_MAX; ++i) {
    po.inbox[i] = reinterpret_cast<__half*>(peers->inbox[i]);
    po.flag[i] = peers->flag[i];
  }
  po.sent = peers->sent;
  po.ticket = peers->ticket;
  po.tp = peers->tp;
  po.rank = peers->rank;
  po.rows_cap = peers->rows_cap;
  po.rows_per = 0;
  moe_combine_kernel<<<rows, 256, 0, stream>>>(expert_out, slots, probs, top_k, shared_out,
                                               shared_gate, nullptr, hidden, po);
  return static_cast<int>(cudaGetLastError());
}

int orinfer_moe_combine(const __half* expert_out, const int* slots, const float* probs, int rows,
                        int top_k, const __half* shared_out, const float* shared_gate,
                        __half* out, int hidden, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden % 8) return -1;
  moe_combine_kernel<<<rows, 256, 0, stream>>>(expert_out, slots, probs, top_k, shared_out,
                                               shared_gate, out, hidden, PeerOut{});
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"
