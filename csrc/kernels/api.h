// C ABI of liborinfer_kernels.so.  Every entry point takes raw device pointers and
// the CUDA stream to launch on, returns 0 on success, a negative value for a
// rejected argument, or the cudaError_t of the launch.  None of them synchronises.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- runtime
int orinfer_init(void);                      // per-device tables + status word (idempotent)
int orinfer_read_status(int* out4);          // synchronises the device; copies 4 ints
int orinfer_clear_status(void);
const void* orinfer_e8p_tables_device(void); // device address of the decode tables
int orinfer_e8p_basis_host(int8_t* out256x8);

// ---- fused tensor-parallel plumbing (all pointers are device addresses; peers' buffers
// are peer-mapped into this process).  tp <= 8.
typedef struct OrinferPeerOut {
  void* inbox[8];              // every rank's inbox for this op: fp16 [tp][rows_cap][n]
  int* flag[8];                // every rank's flag array for this op: int32 [tp]
  int* sent;                   // local sequence counter (device memory)
  unsigned int* ticket;        // local CTA counter (device memory, zero)
  int tp, rank, rows_cap;
  int rows_per;                // 0: push every row to every rank (all-reduce);
                               // > 0: row m only to rank m / rows_per (reduce-scatter);
                               // -1: low-latency all-reduce (<= 8 rows, Q4/Q2 weights): inbox[]
                               //     are the LL regions, sent / ticket the LL counters
} OrinferPeerOut;

// Sequence-parallel all-gather by push (see tp_comm.cuh).
typedef struct OrinferAgOut {
  void* q[8];                  // every rank's activation buffer: int8 [rows_cap][K]
  float* scale[8];             // every rank's row scales: fp32 [rows_cap]
  int* flag[8];                // every rank's all-gather flags: int32 [tp]
  int* sent;                   // local sequence counter (device memory)
  unsigned int* ticket;        // local CTA counter (device memory, zero)
  int tp, rank, rows_per;
} OrinferAgOut;

typedef struct OrinferAgIn {
  const int* flag;             // local all-gather flags
  const int* sent;             // local sequence counter of the producing norm kernel
  int tp, rows_per;
} OrinferAgIn;



typedef struct OrinferInbox {
  const void* inbox;           // local inbox: fp16 [tp][rows_cap][n]
  const int* flag;             // local flag array: int32 [tp]
  int* seen;                   // local sequence counter (device memory)
  unsigned int* ticket;        // local CTA counter (device memory, zero)
  int tp, rows_cap;
  const void* ll;              // non-null: low-latency form (<= 8 rows): uint2 [tp][8][n / 2]
                               // units {2 x fp16, sequence number}; seen / ticket are its counters
} OrinferInbox;

// Cross-rank merge of a vocabulary-sharded head's greedy token (tp_head.cu).
typedef struct OrinferHeadMerge {
  void* table[8];              // every rank's table: uint4 [tp][cap], zero-initialised
  int* seq;                    // local sequence counter (device memory)
  int tp, rank, cap;
} OrinferHeadMerge;
int orinfer_tp_head_merge(const float* logits, const int* local_tok, int rows, int vocab_local,
                          int vocab0, const OrinferHeadMerge* h, int* token_out,
                          cudaStream_t stream);

// Owner rows [rank*rows_per, ...) only: sum the tp partial rows of the inbox, add the
// residual, normalise, rotate, quantise, store the INT8 row + scale into every rank's
// activation buffer and publish the all-gather flag.
int orinfer_act_prep_sp(const OrinferInbox* inbox, const OrinferAgOut* ag, float* resid,
                        const __half* norm_w, const int8_t* signs, int rows, int K, float eps,
                        int zero_centered, cudaStream_t stream, const __half* x);
int orinfer_act_prep_inbox_rows(const OrinferInbox* inbox, float* resid, const __half* norm_w,
                                const int8_t* signs, int8_t* q_out, float* scale_out,
                                __half* y_out, int row_base, int count, int K, float eps,
                                int zero_centered, cudaStream_t stream);
// Column-parallel GEMM whose A operand (and row scales) is the all-gathered activation
// buffer: waits per M tile for the source ranks' flags before loading.
int orinfer_qgemm_ag(int fmt, const int8_t* a, const float* a_scale, const void* w,
                     const __half* w_scale, void* out, const OrinferAgIn* ag, int M, int N, int K,
                     int out_f32, cudaStream_t stream);
// Waits (bounded) for every source of the current all-gather; later kernels on the stream
// may then read the activation buffer with ordinary loads.
int orinfer_ag_wait(const OrinferAgIn* ag, int rows, cudaStream_t stream);

int orinfer_act_prep_limited(const __half* x, const int8_t* signs, int8_t* q_out,
                             float* scale_out, int rows, int K, int swiglu, const int* row_limit,
                             cudaStream_t stream);
int orinfer_act_prep_inbox(const OrinferInbox* inbox, float* resid, const __half* norm_w,
                           const int8_t* signs, int8_t* q_out, float* scale_out, __half* y_out,
                           int rows, int K, float eps, int zero_centered, cudaStream_t stream);
// Row-parallel projection whose FP16 partial result goes to slot [rank] of every peer's
// inbox instead of a local matrix (GEMM fused with the scatter half of an all-reduce).
int orinfer_qgemm_peer(int fmt, const int8_t* a, const float* a_scale, const void* w,
                       const __half* w_scale, const OrinferPeerOut* peer, int M, int N, int K,
                       int force_path, cudaStream_t stream);

// ---- peer-mapped buffers (CUDA IPC, one node)
void* orinfer_peer_alloc(size_t bytes);
int orinfer_peer_free(void* p);
int orinfer_peer_export(void* p, unsigned char* handle64);
int orinfer_peer_import(const unsigned char* handle64, void** out);
int orinfer_peer_unmap(void* p);
int orinfer_peer_copy(void* dst, const void* src, size_t bytes);

// ---- row kernels
int orinfer_embed_w8(const int* ids, const int8_t* table, const __half* scales, __half* out,
                     int rows, int hidden, int vocab, cudaStream_t stream);
int orinfer_act_prep(const __half* x, float* resid, const __half* norm_w, const int8_t* signs,
                     int8_t* q_out, float* scale_out, __half* y_out, int rows, int K, float eps,
                     int zero_centered, int swiglu, cudaStream_t stream);
int orinfer_rope_table(const int* positions, float* cosb, float* sinb, int rows, int head_dim,
                       double theta, cudaStream_t stream);
int orinfer_qk_rope_kv(const __half* qkv, const __half* wq, const __half* wk, const float* cosb,
                       const float* sinb, const int* row_req, const int* row_pos,
                       const int* page_table, int max_pages, int rows, int qh, int kvh,
                       int head_dim, int gated, float eps, int zero_centered, __half* q_out,
                       __half* gate_out, int8_t* kcache, int8_t* vcache, __half* kscale,
                       __half* vscale, int num_pages, cudaStream_t stream);
int orinfer_argmax_parts(int vocab);
int orinfer_argmax(const float* logits, int rows, int vocab, float* scratch_val, int* scratch_idx,
                   int* token, cudaStream_t stream);

// ---- quantised GEMM.  fmt: 0 = W8 [N,K] int8, 1 = E8P Q4 U32 [K/128,N,16], 2 = E8P Q2 U16
// [K/128,N,16].  out is fp16 [M,N] (out_f32 = 0) or fp32.  out[m,n] = acc * s_w[n] * s_a[m].
int orinfer_qgemm(int fmt, const int8_t* a, const float* a_scale, const void* w,
                  const __half* w_scale, void* out, int M, int N, int K, int out_f32,
                  int force_path, cudaStream_t stream);

// ---- mixture of experts
int orinfer_router_topk(const __half* x, const __half* w, int rows, int hidden, int experts,
                        int has_shared, int top_k, int renorm, int* ids, float* probs,
                        float* shared_gate, cudaStream_t stream);
int orinfer_moe_dispatch(const int* ids, int rows, int top_k, int experts, const int8_t* q8,
                         const float* scale, int K, int* counts, int* offsets, int* tiles,
                         int* meta, int max_tiles, int* slots, int8_t* q8_sorted,
                         float* scale_sorted, cudaStream_t stream);
int orinfer_moe_combine(const __half* expert_out, const int* slots, const float* probs, int rows,
                        int top_k, const __half* shared_out, const float* shared_gate,
                        __half* out, int hidden, cudaStream_t stream);
int orinfer_moe_dispatch_ep(const int* ids, int rows, int top_k, int base_expert,
                            int local_experts, const int8_t* q8, const float* scale, int K,
                            int* counts, int* offsets, int* tiles, int* meta, int max_tiles,
                            int* slots, int8_t* q8_sorted, float* scale_sorted,
                            cudaStream_t stream);
int orinfer_moe_combine_peer(const __half* expert_out, const int* slots, const float* probs,
                             int rows, int top_k, const __half* shared_out,
                             const float* shared_gate, const OrinferPeerOut* peers, int hidden,
                             cudaStream_t stream);
int orinfer_qgemm_launches(int M, int N, int K, int out_f32, int force_path);
int orinfer_qgemm_launches_fmt(int fmt, int M, int N, int K, int out_f32, int force_path);
int orinfer_qgemm_set_variant(int fmt, int m_lo, int m_hi, int n, int k, int mt, int nb,
                              int splits);
void orinfer_qgemm_clear_variants();
void orinfer_qgemm_plan(int fmt, int M, int N, int K, int out_f32, int* out);
int orinfer_qgemm_grouped(int fmt, const int8_t* a, const float* a_scale, const void* w,
                          const __half* w_scale, void* out, int S, int N, int K, int experts,
                          const int* tiles, const int* meta, int max_tiles, cudaStream_t stream);

// ---- attention over the paged INT8 KV cache
size_t orinfer_attention_scratch_bytes(int rows, int qh, int head_dim, int splits);
int orinfer_attention(const __half* q, const __half* gate, const int* row_req, const int* row_pos,
                      const int* page_table, int max_pages, const int8_t* kcache,
                      const int8_t* vcache, const __half* kscale, const __half* vscale,
                      __half* out, int rows, int qh, int kvh, int head_dim, int splits,
                      float* scratch, cudaStream_t stream);

// Prefill chunks on tensor cores.  chunks: device int32 [n_chunks, 4] =
// (first packed row, rows, absolute position of the first row, page-table row).
// Returns -4 for a head size it does not implement (use orinfer_attention instead).
int orinfer_attention_prefill(const __half* q, const __half* gate, const int* chunks, int n_chunks,
                              int max_q_len, int total_rows, const int* page_table, int max_pages,
                              const int8_t* kcache, const int8_t* vcache, const __half* kscale,
                              const __half* vscale, __half* out, int qh, int kvh, int head_dim,
                              int num_pages, cudaStream_t stream);

// ---- expert-parallel all-to-alls over peer memory (moe_a2a.cu); cap = owned rows x top_k
typedef struct OrinferA2aDispatch {
  void* rows[8];               // every rank's receive buffer: int8 [tp][cap][K]
  float* scale[8];             // fp32 [tp][cap]
  int* expert[8];              // int32 [tp][cap]
  int* header[8];              // int32 [tp][2] = (count, base slot at the sender)
  int* flag[8];                // int32 [tp]
  int* sent;                   // local sequence counter
  unsigned int* ticket;        // local CTA counter
  int tp, rank, cap;
} OrinferA2aDispatch;

typedef struct OrinferA2aReturn {
  void* ret[8];                // every rank's return buffer: fp16 [cap][H]
  int* flag[8];
  int* sent;
  unsigned int* ticket;
  int tp, rank, cap;
} OrinferA2aReturn;

int orinfer_a2a_dispatch_push(const int* ids, const int* slots, const int* offsets,
                              const int8_t* q8, const float* scale, int rows, int top_k, int K,
                              int experts_per_rank, const OrinferA2aDispatch* d,
                              cudaStream_t stream);
int orinfer_a2a_recv_prepare(const int* flag, const int* sent, const int* header, int* expert,
                             int tp, int cap, cudaStream_t stream);
int orinfer_a2a_return_push(const __half* down, const int* slots, const int* header, int H,
                            const OrinferA2aReturn* r, cudaStream_t stream);
int orinfer_a2a_wait(const int* flag, const int* sent, int tp, cudaStream_t stream);

// ---- gated-delta-rule linear attention (segments: int32 [n,4] = first row, rows, 0, 0;
// the state slot of a row is row_slot[row]; a segment starting at position 0 starts fresh)
int orinfer_small_proj(const __half* x, const __half* w, float* out, int rows, int hidden, int n,
                       cudaStream_t stream);
int orinfer_gdn_conv(const __half* x, int x_stride, const __half* weight, __half* hist,
                     const int* row_first, const int* row_slot, const int* row_pos,
                     const int* segs, int n_segs, int rows, int hk, int hv, int head_dim, __half* y,
                     cudaStream_t stream, int update_history);
int orinfer_gdn_scan(const __half* qkv, const float* ab, const float* a_log, const float* dt_bias,
                     const int* segs, int n_segs, const int* row_slot, const int* row_pos, int hk,
                     int hv, int head_dim, float* state, float* out, cudaStream_t stream,
                     float* factors);
// factors: fp32 [rows, HV, 2*D + 1] recorded by a scan with factors != NULL (which leaves the
// state untouched); accepted: int32 [n_segs] rows of each segment to keep.
int orinfer_gdn_commit(const __half* x, int x_stride, const float* factors, const int* segs,
                       int n_segs, const int* accepted, const int* row_slot, const int* row_pos,
                       int hk, int hv, int head_dim, __half* hist, float* state,
                       cudaStream_t stream);
int orinfer_gdn_gated_norm(const float* o, const __half* z, int z_stride, const __half* w,
                           float eps, int sigmoid_gate, int rows, int hv, int head_dim,
                           __half* y, cudaStream_t stream);

// ---- device top-k / top-p sampler (rows it cannot serve exactly get flag = 1)
int orinfer_sample_topk(const float* logits, int rows, int vocab, long long row_stride,
                        const int* top_k, const double* temperature, const double* top_p,
                        const double* uniform, int* token, int* flag, cudaStream_t stream);

// ---- E8P nearest-codeword encoder: x fp32 [V,8] -> int32 codes [V]
int orinfer_e8p_encode(const float* x, int* codes, long long vectors, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
