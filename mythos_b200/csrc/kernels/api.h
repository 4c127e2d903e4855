// Raw-pointer launch API of the sm_100a kernel library. No framework types appear here:
// the torch binding (bindings.cpp) and the C ABI both sit on top of these functions.
// All launchers are asynchronous on `stream`, bump the library's launch counter and throw
// std::invalid_argument / mb::CudaError on bad arguments or launch failure.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb {

// ---- GEMM epilogues
enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_F32_ACC = 2, EPI_F32_ATOMIC = 3 };

// C[M,N] (+)= alpha * A * B^T on tcgen05 tensor cores. a_mn / b_mn: operand is stored
// transposed ([K,M] / [K,N] row-major). lda/ldb/ldc are row strides in elements.
// `status` (device int, may be null) receives a non-zero code if a bounded wait expires.
void gemm_bf16(const void* A, long long lda, bool a_mn, const void* B, long long ldb, bool b_mn, void* C,
               long long ldc, int M, int N, int K, int epi, float alpha, int* status, cudaStream_t stream);

// Paired-SM variant (cta_group::2, 256x256 tile per 2-CTA cluster); same contract.
void gemm_bf16_2cta(const void* A, long long lda, bool a_mn, const void* B, long long ldb, bool b_mn, void* C,
                    long long ldc, int M, int N, int K, int epi, float alpha, int* status, cudaStream_t stream);
struct PeerPtrs;
// Same kernel with a fused reduce-scatter epilogue (bf16): output row m goes to rank m / rows_per_rank,
// at scatter[rank] + slot_off + (m % rows_per_rank) * ldc, a peer store from the epilogue.
void gemm_bf16_2cta_scatter(const void* A, long long lda, bool a_mn, const void* B, long long ldb, bool b_mn, void* C,
                            long long ldc, int M, int N, int K, int epi, float alpha, int* status,
                            cudaStream_t stream, const PeerPtrs* scatter, int n_scatter, long long rows_per_rank,
                            long long slot_off);
// Work folded into the paired kernel's epilogue (gemm_2cta.cu).
enum : int { FUSE_NONE = 0, FUSE_SWIGLU_FWD = 1, FUSE_SWIGLU_BWD = 2, FUSE_ROPE = 3 };
struct EpiFuse {
  int F = 0;                              // SwiGLU: ffn width (number of gate columns)
  const __nv_bfloat16* aux = nullptr;     // SWIGLU_BWD: saved gate|up pre-activations [M, 2F]
  long long ld_aux = 0;
  __nv_bfloat16* out2 = nullptr;          // SWIGLU_FWD: h = silu(gate) * up, [M, F]
  long long ld_out2 = 0;
  const int* pos = nullptr;               // ROPE: position of every row
  const float2* cs = nullptr;             // ROPE: [max_pos, 64] (cos, sin) of pair j at angle pos * theta^(-2j/128)
  int max_pos = 0;
  int rope_cols = 0;                      // ROPE: columns [0, rope_cols) are rotated heads of 128
};
// gate_up[M, 2F] (may be null) and h[M, F] = silu(gate) * up from x[M, K] and the fused [2F, K] weight
// (gate rows first), one launch; F must be a multiple of 128.
void gemm_swiglu_fwd(const void* x, long long ldx, const void* w_gate_up, long long ldw, void* gate_up, long long ld_gu,
                     void* h, long long ld_h, int M, int F, int K, int* status, cudaStream_t stream);
// d_gate_up[M, 2F] from dy[M, K], the down-projection weight [K, F] and the saved pre-activations:
// the dgrad GEMM dh = dy W_down with the SwiGLU backward applied in the epilogue.
void gemm_swiglu_bwd(const void* dy, long long ld_dy, const void* w_down, long long ldw, const void* gate_up,
                     long long ld_gu, void* d_gate_up, long long ld_dgu, int M, int F, int K, int* status,
                     cudaStream_t stream);
// out[M, N] = x[M, K] w[N, K]^T with the half-split rotary embedding applied to the heads (128 columns
// each) in columns [0, rope_cols); cos_sin is the [max_pos, 64, 2] fp32 table.
void gemm_rope(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo, int M, int N, int K,
               const int* pos, const float* cos_sin, int max_pos, int rope_cols, int* status, cudaStream_t stream);
// Grouped (ragged) GEMMs on the paired kernel: one launch over up to 16 segments of a row-indexed buffer
// (the tokens routed to each local expert). seg_start / seg_rows are DEVICE arrays of n_seg ints; starts
// are multiples of 256 and the rows from a segment's end up to the next multiple of 256 must hold zeros.
//   rows: C[rows of e, 0:N] = A[rows of e, 0:K] * B[e]^T with B[e] = [N, K] (or [K, N] with b_mn). `fuse`:
//         FUSE_NONE, FUSE_SWIGLU_FWD (N = 2F; C = pre-activations or null, out2 = h[rows, F]) or
//         FUSE_SWIGLU_BWD (B[e] = [K, F] read MN-major, aux = pre-activations, C = d pre-activations [rows, 2F]).
//   k:    C[e][M, N] += A[rows of e, 0:M]^T * B[rows of e, 0:N] in fp32 (weight gradients).
// B / C are HOST arrays of device pointers.
void gemm_grouped_rows(const void* A, long long lda, int total_rows, const void* const* B, long long ldb, bool b_mn,
                       void* C, long long ldc, int N, int K, const int* seg_start, const int* seg_rows, int n_seg,
                       int fuse, const void* aux, long long ld_aux, void* out2, long long ld_out2, int* status,
                       cudaStream_t stream);
void gemm_grouped_k(const void* A, long long lda, const void* B, long long ldb, float* const* C, long long ldc, int M,
                    int N, int total_rows, const int* seg_start, const int* seg_rows, int n_seg, int* status,
                    cudaStream_t stream);
double gemm_2cta_waves(int M, int N, int sms);
// 1 (default): the paired kernel's plain epilogues store through a shared-memory transpose; 0: from registers.
void set_gemm_coalesced_epilogue(int on);
// 0 = choose per problem, 1 = always the single-CTA kernel, 2 = the paired kernel whenever it applies.
void set_gemm_mode(int mode);
int get_gemm_mode();

// ---- normalisation (norm.cu)
void rmsnorm_fwd(const void* x, const void* residual, const void* gamma, void* y, void* resid_out, float* rstd,
                 int rows, int dim, float eps, cudaStream_t stream);
// dres (bf16 [rows, dim], may be null): gradient arriving through the residual stream, added to dx.
void rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx, float* dgamma_partial,
                 int rows, int dim, int n_partial, cudaStream_t stream, const void* dres = nullptr);
void rmsnorm_bwd_reduce(const float* dgamma_partial, float* dgamma, int n_partial, int dim, bool accumulate,
                        cudaStream_t stream);
void layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, int rows, int dim, float eps,
                   cudaStream_t stream);
// dx and per-CTA partials [n_partial, 2 * dim] = [dgamma | dbeta]; mean / rstd are recomputed from x.
void layernorm_bwd(const void* dy, const void* x, const void* gamma, void* dx, float* partial, int n_partial, int rows,
                   int dim, float eps, cudaStream_t stream);

// ---- rotary embedding, half-split pairs (d, d + D/2) (rope.cu)
// x: [tokens, heads, head_dim] bf16 in place; pos: [tokens] int32; inverse = backward pass.
void rope_apply(void* x, const int* pos, int tokens, int heads, int head_dim, long long token_stride, float theta,
                bool inverse, cudaStream_t stream);

// ---- activations / pointwise (act.cu)
void swiglu_fwd(const void* gate, const void* up, void* out, long long n, cudaStream_t stream);
void swiglu_bwd(const void* gate, const void* up, const void* dout, void* dgate, void* dup, long long n,
                cudaStream_t stream);
// gate/up interleaved in one [rows, 2*ffn] buffer (gate = cols [0,ffn), up = cols [ffn,2ffn))
void swiglu_fused_fwd(const void* gate_up, void* out, long long rows, int ffn, cudaStream_t stream);
void swiglu_fused_bwd(const void* gate_up, const void* dout, void* dgate_up, long long rows, int ffn,
                      cudaStream_t stream);
void relu2_fwd(const void* x, void* out, long long n, cudaStream_t stream);
void relu2_bwd(const void* x, const void* dout, void* dx, long long n, cudaStream_t stream);
enum : int { ACT_RELU = 0, ACT_GELU_ERF = 1, ACT_GELU_TANH = 2, ACT_SILU = 3, ACT_SIGMOID = 4, ACT_TANH = 5 };
void act_fwd(const void* x, void* out, long long n, int kind, cudaStream_t stream);
void act_bwd(const void* x, const void* dout, void* dx, long long n, int kind, cudaStream_t stream);
void add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream);
void softmax_rows(const void* x, void* y, int rows, int cols, cudaStream_t stream);
void softmax_rows_bwd(const void* y, const void* dy, void* dx, int rows, int cols, cudaStream_t stream);

// ---- embedding (embed.cu)
void embedding_fwd(const int* ids, const void* table, void* out, int tokens, int dim, int vocab, cudaStream_t stream);
void embedding_bwd(const int* ids, const void* dout, float* dtable, int tokens, int dim, int vocab, cudaStream_t stream);

// ---- cross-entropy: per-row loss + in-place gradient (ce.cu)
// logits [rows, vocab] bf16 is overwritten with (softmax - onehot) * grad_scale; losses [rows] fp32.
void cross_entropy_fwd_bwd(void* logits, const int* targets, float* losses, int rows, int vocab, long long ld,
                           float grad_scale, cudaStream_t stream);
void cross_entropy_fwd(const void* logits, const int* targets, float* losses, int rows, int vocab, long long ld,
                       cudaStream_t stream);
// Vocabulary-parallel form: this rank holds logits columns [vocab_offset, vocab_offset + vocab).
// stats[row] = {local max, local sum exp(x - max), target logit or 0}; after the ranks have merged
// the records into lse[row], the second call overwrites the local logits with their gradient.
void cross_entropy_shard_stats(const void* logits, const int* targets, float* stats, int rows, int vocab, long long ld,
                               int vocab_offset, int vocab_total, cudaStream_t stream);
void cross_entropy_shard_grad(void* logits, const int* targets, const float* lse, int rows, int vocab, long long ld,
                              int vocab_offset, int vocab_total, float grad_scale, cudaStream_t stream);

// ---- optimizer + STE fake-quant (optim.cu, quant.cu)
struct AdamWArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale;
};
// p/m/v fp32 master state, g fp32 gradient (scaled by grad_scale and, when clip_coef is non-null,
// by *clip_coef read on the device); optional bf16 shadow copy of p written to p_bf16.
void adamw_step(float* p, float* m, float* v, const float* g, void* p_bf16, long long n, AdamWArgs a,
                const float* clip_coef, cudaStream_t stream);
void sumsq_f32(const float* x, long long n, float* out_accum, cudaStream_t stream);
// Nearest-centroid fake quantisation through sorted codebooks.
// w fp32 [n]; block b (bs weights) uses codebook cb_map[b] (or b when cb_map is null) of
// `cb_size` ascending fp32 centroids. Outputs: bf16 dequantised weight and/or u8 indices.
void oil_fake_quant(const float* w, const float* codebooks, const int* cb_map, int cb_size, int bs, long long n,
                    void* w_bf16, uint8_t* idx, cudaStream_t stream);
// I2_S ternary: per-block absmean scale, trit = clamp(round(w/scale), -1, 1).
void i2s_fake_quant(const float* w, int bs, long long n, void* w_bf16, uint8_t* trits, float* scales,
                    cudaStream_t stream);
void cast_f32_to_bf16(const float* x, void* y, long long n, cudaStream_t stream);
void cast_bf16_to_f32(const void* x, float* y, long long n, bool accumulate, cudaStream_t stream);
// Codebook EMA statistics: counts[cb, k] += 1, sums[cb, k] += w for each weight's centroid.
void oil_codebook_stats(const float* w, const uint8_t* idx, const int* cb_map, int cb_size, int bs, long long n,
                        float* counts, float* sums, cudaStream_t stream);

// ---- flash attention, training (attention.cu)
// q,k,v,o: [batch, seq, heads, head_dim] bf16 (k/v with kv_heads); lse: [batch, heads, seq] fp32.
void flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq, int heads,
                    int kv_heads, int head_dim, bool causal, float scale, int* status, cudaStream_t stream);
void flash_attn_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq,
                            int heads, int kv_heads, int head_dim, long long q_tok_stride, long long kv_tok_stride,
                            long long o_tok_stride, bool causal, float scale, int* status, cudaStream_t stream);
// Second-generation forward for head_dim 128 (attention_fwd2.cu): persistent CTAs, 128 x 128 score tiles, P in
// tensor memory. set_attn_fwd_mode(1) routes flash_attn_fwd / _strided to it where it applies (0: first kernel).
bool flash_attn_fwd2_supported(int head_dim, int seq);
void flash_attn_fwd2_strided(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq,
                             int heads, int kv_heads, long long q_tok_stride, long long kv_tok_stride,
                             long long o_tok_stride, bool causal, float scale, int* status, cudaStream_t stream);
void set_attn_fwd_mode(int mode);
int get_attn_fwd_mode();
// Prefill attention over the paged KV cache (tcgen05, causal): q holds the NEW tokens of `batch` sequences
// packed back to back (sequence b = rows cu_q[b] .. cu_q[b+1]); k_cache / v_cache are bf16 pages
// [n_pages, 16, kv_heads, head_dim] addressed through block_table [batch, table_stride]; kv_lens[b] counts the
// keys the last query of b sees (cached prefix + new tokens, which must already be in the pages).
void flash_attn_paged_prefill(const void* q, long long q_tok_stride, const void* k_cache, const void* v_cache,
                              int n_pages, const int* block_table, int table_stride, const int* cu_q, const int* kv_lens,
                              void* o, long long o_tok_stride, int batch, int total_q, int max_q_len, int heads,
                              int kv_heads, int head_dim, float scale, int* status, cudaStream_t stream);
void flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                    void* dq, void* dk, void* dv, float* dq_accum, float* delta, int batch, int seq, int heads,
                    int kv_heads, int head_dim, bool causal, float scale, int* status, cudaStream_t stream);
void flash_attn_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* dout,
                            const float* lse, void* dq, void* dk, void* dv, float* dq_accum, float* delta, int batch,
                            int seq, int heads, int kv_heads, int head_dim, long long q_tok_stride,
                            long long kv_tok_stride, long long dq_tok_stride, long long dkv_tok_stride, bool causal,
                            float scale, int* status, cudaStream_t stream, const int* rope_pos = nullptr,
                            const float* rope_cs = nullptr, int rope_max_pos = 0);
// rope_cs ([rope_max_pos, 64, 2] fp32 cos/sin) with rope_pos ([batch * seq] int32): q and k were rotated
// before the forward pass, and dq / dk leave rotated back (dq in the fp32 -> bf16 conversion, dk in the
// kernel's epilogue), i.e. as gradients of the un-rotated projection.

// ---- fused decode epilogues (decode_fused.cu)
// Exactly one of `acc` (fp32 [rows, dim], zeroed) / `slots` (n_slots bf16 partials, slot_stride apart) is summed,
// `residual` (may be null) is added, the bf16 result goes to stream_out and its RMS-normalised image to normed.
void sum_residual_rmsnorm(float* acc, const void* slots, int n_slots, long long slot_stride, const void* residual,
                          const void* gamma, void* stream_out, void* normed, int rows, int dim, float eps,
                          cudaStream_t stream);
// Tensor-parallel form: pushes this rank's partial row (acc, may be null when the GEMM stored the slots)
// into slot `rank` of every rank's staging buffer, signals and awaits per-row flags
// (flags: int32 [2][world][max_rows] per rank), then sums the world's slots + residual and normalises.
// epoch_dev / arrive: one int each in local device memory, both zero before the first call.
void tp_sum_residual_rmsnorm(float* acc, const PeerPtrs& staging, const PeerPtrs& flags, int rank, int world,
                             long long slot_stride, int parity, int max_rows, const void* residual, const void* gamma,
                             void* stream_out, void* normed, int rows, int dim, float eps, int* epoch_dev, int* arrive,
                             long long limit_cycles, int* status, cudaStream_t stream);
// acc fp32 [tokens, (heads + 2 kv_heads) * head_dim] (zeroed): Q rotated -> q_out bf16 [tokens, heads, head_dim];
// K rotated and V -> their cache pages. theta <= 0 disables the rotation.
void qkv_rope_append(float* acc, const int* pos, const int* seq_ids, const int* block_table, void* q_out,
                     void* k_cache, void* v_cache, int tokens, int heads, int kv_heads, int head_dim, int page_size,
                     int max_pages, float theta, cudaStream_t stream, float* k_scale = nullptr,
                     float* v_scale = nullptr);   // scales given: k_cache / v_cache are int8 pages
// acc fp32 [rows, 2 * ffn] (zeroed) -> act(gate) * up, bf16 [rows, ffn]; kind 0 SiLU, 1 squared ReLU.
void finalize_gate(float* acc, void* out, long long rows, int ffn, int kind, cudaStream_t stream);

// ---- ternary look-up-table GEMMs with int8 activations (ternary_lut.cu)
// y[M, N] fp32 = TL1 (group 2) / TL2 (group 3) product of x[M, K] fp32 with packed trits [N, K / 4].
void tl_gemm(const uint8_t* packed, const float* x, float* y, int M, int N, int K, int group, cudaStream_t stream);

// ---- peer-memory collectives fused with compute (comm.cu)
constexpr int MAX_PEERS = 16;
struct PeerPtrs {
  void* p[MAX_PEERS];  // the same symmetric buffer as mapped on this rank, one pointer per rank
};
enum : int { ZERO_FMT_CAST = 0, ZERO_FMT_OIL8 = 1, ZERO_FMT_OIL4 = 2, ZERO_FMT_I2S = 3, ZERO_FMT_BINARY = 4 };
struct ZeroFusedArgs {
  float *p, *m, *v;            // local fp32 shard of master weights and Adam moments, n elements
  const float* g;              // local reduced gradient shard
  PeerPtrs compute;            // every rank's full bf16 compute buffer
  void* compute_mc = nullptr;  // NVLS multicast address of the compute buffers (null: plain peer stores)
  long long shard_off, n;      // element offset of the shard in the flat buffer; shard length
  const uint8_t* seg_fmt;      // per 256-element segment of the flat buffer: ZERO_FMT_*
  const int* seg_cb;           // per segment: codebook row in codebooks8 / codebooks4
  const float* codebooks8;     // [n, 256] ascending fp32
  const float* codebooks4;     // [n, 16] ascending fp32
  const float* norm_partials;  // world floats: each rank's sum of squares of its reduced shard
  float* grad_norm_out;        // optional: the global gradient norm
  float max_norm;              // clip threshold (0 = off)
  AdamWArgs opt;
  int rank, world;
};
// Flag barrier across ranks; with send_val != null also delivers *send_val into slot [rank] of every
// rank's `slots` array. The wait gives up after limit_cycles and records it in `status`.
// With epoch_ptr != null the epoch is read from (and advanced in) device memory instead of `epoch`.
void symm_barrier(const PeerPtrs& flags, const PeerPtrs& slots, const float* send_val, int rank, int world, int epoch,
                  int* epoch_ptr, long long limit_cycles, int* status, cudaStream_t stream);
// out = {barriers launched, sum of wait cycles, longest wait in cycles} on the current device since the
// last reset (SM clock cycles between a rank's arrival and the last peer's); synchronises the device.
void comm_barrier_wait_stats(unsigned long long out[3], bool reset);
// All-gather of a row-sharded A fused into the GEMM C = A B^T (gemm_2cta.cu, GROUP_GATHER): copier CTAs of
// the same launch pull the peers' rows into a_bufs.p[rank] with non-multicast TMA copies while the other
// SM pairs multiply, own rows first. M % (256 * world) == 0, K % 64 == 0, world <= 8.
void gemm_allgather_a(const PeerPtrs& a_bufs, long long lda, const void* B, long long ldb, void* C, long long ldc, int M,
                      int N, int K, int rank, int world, int* tile_count, int call, int copier_clusters, int* status,
                      cudaStream_t stream);
// The weight-side form: B [N, K] sharded by rows over the ranks (a sharded bf16 compute image), gathered into
// b_bufs.p[rank] by copier CTAs of the launch while the other SM pairs multiply, own column block first.
// N % (256 * world) == 0, K % 64 == 0, world <= 8.
void gemm_allgather_b(const void* A, long long lda, const PeerPtrs& b_bufs, long long ldb, void* C, long long ldc, int M,
                      int N, int K, int rank, int world, int* tile_count, int call, int copier_clusters, int* status,
                      cudaStream_t stream);
// Registers the status word of the current device: the kernels below that consume data guarded by a
// flag barrier (zero_reduce_scatter, zero_adamw_ste_allgather, tp_reduce_slots, tp_reduce_slots_bcast,
// tp_allreduce_pull) return without writing once the word is non-zero (a bounded wait expired).
void comm_set_abort_word(const int* status);
// block_partials (zeroed fp32 scratch of n_block_partials >= 2 words, not shared by launches that can run at
// the same time): the sum of squares is then added in a fixed order and is bit-reproducible.
// grads_multicast: NVLS multicast address of the gradient buffers (the sum is then formed inside the
// NVSwitch by multimem.ld_reduce; null: one peer load per rank, added in rank order). max_blocks > 0 caps the grid.
void zero_reduce_scatter(const PeerPtrs& grads, float* out, long long shard_off, long long n, int world, float* sumsq,
                         cudaStream_t stream, const float* grads_multicast = nullptr, int max_blocks = 0,
                         float* block_partials = nullptr, long long n_block_partials = 0);
// All-reduce of bf16 partials through NVLS (multimem.ld_reduce + multimem.st on multicast addresses):
// this rank handles slice `rank` of n elements; barriers before and after are the caller's.
void tp_allreduce_multimem(const void* part_mc, void* out_mc, int n_peers, int rank, long long n, cudaStream_t stream);
void zero_adamw_ste_allgather(const ZeroFusedArgs& a, cudaStream_t stream);
// dst_r[i] += part[i] on every rank r (fp32 peer reductions).
void peer_add_f32(const float* part, const PeerPtrs& dst, int n_peers, long long n, cudaStream_t stream);
// Column all-gather by peer stores: dst_r[b, rank*cols + j] = src[b, j] on every rank r.
// Tensor-parallel all-reduce building blocks (bf16 activations, see comm.cu).
void tp_push(float* acc, const PeerPtrs& dst, int n_peers, int rank, long long slot_off, long long n,
             cudaStream_t stream);
void tp_reduce_slots(const void* staging, int slots, long long slot_stride, const void* residual, void* out,
                     long long n, cudaStream_t stream);
void tp_allreduce_pull(const PeerPtrs& part, const PeerPtrs& out, int n_peers, int rank, long long n,
                       cudaStream_t stream);
// Reduce-scatter by peer loads: out_local[0 : n / n_peers) = sum over ranks of part_q[rank * n / n_peers + i].
void tp_reduce_scatter_pull(const PeerPtrs& part, int n_peers, int rank, long long n, void* out_local,
                            cudaStream_t stream);
// Second half of the fused GEMM -> reduce-scatter: sum the `slots` partials of this rank's rows
// (local staging) and store the bf16 result at out_p + out_off for every peer p (all-gather by stores).
void tp_reduce_slots_bcast(const void* staging, int slots, long long slot_stride, const PeerPtrs& out, int n_peers,
                           int rank, long long out_off, long long n, cudaStream_t stream);
void peer_gather_cols(const void* src, const PeerPtrs& dst, int n_peers, int rank, long long rows, int cols,
                      cudaStream_t stream);

// ---- inference: codebook-dequant GEMM (dequant_gemm.cu)
enum : int { QFMT_OIL8 = 3, QFMT_OIL4 = 2, QFMT_I2S = 1 };  // numeric values of the container's Format enum
struct DequantWeights {
  const uint8_t* packed;     // OIL8: N*K bytes; OIL4: N*K/2 (even index in the low nibble); I2_S: N*K/4 (LSB first)
  const void* codebooks;     // bf16 [n_cb, 256] (OIL8) or [n_cb, 16] (OIL4); unused for I2_S
  const int* cb_map;         // per block: codebook row (null = block index)
  const float* scales;       // I2_S: per-block scale
  int fmt, N, K, block_size; // blocks run along K inside a row; K % block_size == 0
  int n_codebooks;           // rows of `codebooks`
};
// y = x * dequant(W)^T. Exactly one output: out_bf16 (no split-K), or fp32 accumulation into
// out_f32 / into every buffer of `peers` (fused all-reduce; buffers must hold zeros or a residual).
// k_splits <= 0 picks enough splits to fill the GPU.
void dequant_gemm(const void* x, long long ldx, int M, const DequantWeights& w, void* out_bf16, float* out_f32,
                  const PeerPtrs* peers, int n_peers, long long ld_out, int k_splits, int* status, cudaStream_t stream,
                  long long peer_bf16_offset = -1);
// out = bf16(acc (+ residual)); acc is reset to zero for its next accumulation.
void finalize_acc(float* acc, const void* residual, void* out, long long n, cudaStream_t stream);
// Whole-matrix dequantisation into a bf16 scratch buffer (prefill path).
void dequant_to_bf16(const DequantWeights& w, void* out, cudaStream_t stream);
// Embedding gather through the quantised table: out[t, :K] = dequant(W[clamp(ids[t]), :]).
void dequant_gather_rows(const DequantWeights& w, const int* ids, int tokens, void* out, long long ld_out,
                         cudaStream_t stream);

// ---- inference: paged KV cache, decode attention, sampler (paged_attn.cu, sampler.cu)
// Cache layout: k_cache / v_cache [num_pages, page_size, kv_heads, head_dim] bf16;
// block_table [batch, max_pages] int32 (page index of each logical page of a sequence).
void kv_append(const void* k, const void* v, void* k_cache, void* v_cache, const int* block_table,
               const int* positions, const int* seq_ids, int tokens, int kv_heads, int head_dim, int page_size,
               int max_pages, long long kv_tok_stride, cudaStream_t stream);
// One query token per sequence: q [batch, heads, head_dim]; context_lens [batch]. Split-KV flash
// decoding: partials in `scratch` (>= batch*heads*splits*(head_dim+2) floats), combined in-kernel.
void paged_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                       const int* context_lens, void* out, float* scratch, int* counters, int batch, int heads,
                       int kv_heads, int head_dim, int page_size, int max_pages, int cache_pages, int splits,
                       float scale, int* status, cudaStream_t stream, long long q_tok_stride = 0);
// int8 pages: k_cache / v_cache [num_pages, page_size, kv_heads, head_dim] int8 with one fp32 scale
// (max|x| / 127) per (token, kv head) in k_scale / v_scale [num_pages * page_size, kv_heads].
void kv_append_int8(const void* k, const void* v, void* k_cache, void* v_cache, float* k_scale, float* v_scale,
                    const int* block_table, const int* positions, const int* seq_ids, int tokens, int kv_heads,
                    int head_dim, int page_size, int max_pages, long long kv_tok_stride, cudaStream_t stream);
void paged_attn_decode_int8(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                            const float* v_scale, const int* block_table, const int* context_lens, void* out,
                            float* scratch, int* counters, int batch, int heads, int kv_heads, int head_dim,
                            int page_size, int max_pages, int cache_pages, int splits, float scale, int* status,
                            cudaStream_t stream, long long q_tok_stride = 0);
// Greedy / temperature / top-k / top-p / repetition-penalty sampling of one token per row.
struct SamplerArgs {
  float temperature, top_p, repetition_penalty;
  int top_k;
  unsigned long long seed;
};
void sample_tokens(const void* logits, long long ld, int rows, int vocab, const int* history, int history_len,
                   const unsigned char* allow_mask, SamplerArgs a, int* out_tokens, float* out_logprob, float* scratch,
                   cudaStream_t stream);
// y[n] = sum_k dequant(W)[n,k] * x[k] for one token (CUDA-core GEMV over packed I2_S trits).
void i2s_gemv(const void* x, const DequantWeights& w, void* y, cudaStream_t stream);

// ---- mixture of experts: routing, dispatch / combine exchange (moe.cu)
// Device-side router (no host round trip): softmax + top-k + slots + combine weights + load statistics;
// its backward; the exchange of per-expert counts between ranks; segment offsets of the receive buffer
// (starts aligned to 256 rows for the grouped GEMMs) and zeroing of the alignment padding.
void moe_route(const void* logits, int ld, int T, int E, int k, float* probs, int* topk_idx, int* slot, float* w,
               int* counts, float* psum, cudaStream_t stream);
void moe_route_bwd(const float* probs, const int* topk_idx, const float* dw, const float* coef, int T, int E, int k,
                   void* dlogits, int ld, cudaStream_t stream);
void moe_publish_counts(const int* counts, const PeerPtrs& tables, int world, int E, int rank, cudaStream_t stream);
void moe_offsets(const int* all_counts, int world, int E, int rank, int cap, int* seg_start, int* seg_rows,
                 int* send_base, int* status, cudaStream_t stream, int* send_limit = nullptr);
// send_limit[e] (optional, from moe_offsets): first row of expert e's segment that does not fit into its
// owner's buffer; dispatch skips and combine ignores rows at or past it, so a full buffer drops rows
// (with the status word raised) instead of storing out of bounds.
void moe_zero_pad(const int* seg_start, const int* seg_rows, int n_seg, int dim, void* a, void* b, int cap,
                  cudaStream_t stream);
void moe_topk(const float* probs, int T, int E, int k, int* topk_idx, int* slot, int* counts, cudaStream_t stream);
// Row (t, j) goes to recv[owner(e)] at row rank*cap + send_off[e] + slot[t, j] (optionally scaled).
void moe_dispatch(const void* x, const int* topk_idx, const int* slot, const int* send_off, const float* row_scale,
                  const PeerPtrs& recv, int T, int k, int dim, int experts_per_rank, int rank, long long cap,
                  cudaStream_t stream, const int* send_limit = nullptr);
// out[t] = sum_j w[t,j] * ybuf[owner][row(t,j)] (w null = 1); with dw also dw[t,j] = <dout[t], y row>.
void moe_combine(const PeerPtrs& ybuf, const int* topk_idx, const int* slot, const int* send_off, const float* w,
                 const void* dout, void* out, float* dw, int T, int k, int dim, int experts_per_rank, int rank,
                 long long cap, cudaStream_t stream, const int* send_limit = nullptr);

long long launch_count();

}  // namespace mb
