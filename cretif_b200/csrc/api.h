// The C interface of the kernel library.
//
// Every launcher takes raw device pointers, sizes and the CUDA stream to launch on, and
// returns 0 when the kernel was launched, a negative cretif::Status for arguments it does
// not take, or a positive cudaError_t.  Element types are passed as codes: 0 = float32,
// 1 = bfloat16.  Nothing here allocates device memory.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// out[t, :] = table[ids[t], :] widened to float32.  An id outside [0, V) sets bit 1 of
// *fault and writes zeros.
int cretif_embed_rows(const void* table, int table_dt, const int* ids, float* out, int T, int H,
                      int V, unsigned int* fault, void* stream);

// v = h[src] (+ delta[src]); if write_h, h[src] = v; out[r] = v * weight * rsqrt(mean(v^2)+eps).
// src = rows ? rows[r] : r.  delta may be null.  rows and write_h exclude each other.
int cretif_add_rmsnorm(float* h, const void* delta, int delta_dt, const float* weight, void* out,
                       int out_dt, const int* rows, int R, int H, float eps, int write_h,
                       void* stream);

// act[t, i] = silu(gate) * up; block = 0: gu row = [gate | up]; block = b: groups of b gate
// columns followed by their b up columns.
int cretif_silu_mul(const void* gu, void* act, int dt, int T, int I, int block, void* stream);

// Rotate q and k of every token by its position's angles (pairing 0: (j, j+rot/2),
// 1: (2j, 2j+1)); q in place.  write_cache bit 0: rotated k and v into the block cache;
// bit 1: k rotated in place too (encoding only; with rot_dim 0 and bit 0 it only stores).
int cretif_rope_kv_append(void* qkv, int ld, int dt, const float* cos_t, const float* sin_t,
                          int pairing, int rot_dim, int nh, int nkv, int hd, const int* tok_pos,
                          const int* tok_seq, const int* seq_slot, const int* table,
                          int table_stride, void* kc, void* vc, int bt, int write_cache, int T,
                          unsigned int* fault, void* stream);

// After a decode step: ids <- sampled (if given), positions and lengths + 1.
int cretif_advance_decode(int* tok_ids, int* tok_pos, int* seq_start, const int* sampled, int B,
                          void* stream);

// C[M,N] (= or +=) A[M,K] · W[N,K]^T, 32-bit FMA on the CUDA cores.
int cretif_gemm_simt(const void* A, int a_dt, const void* W, int w_dt, void* C, int c_dt, int M,
                     int N, int K, int lda, int ldw, int ldc, int accumulate, void* stream);

// C[M,N] (= or +=) X[M,K] · W[N,K]^T for M <= 64 rows, bfloat16 operands, streaming W once.
// K and the row strides must be multiples of 8 and the operands 16-byte aligned.
int cretif_gemm_skinny(const void* X, const void* W, void* C, int c_dt, int M, int N, int K,
                       int ldx, int ldw, int ldc, int accumulate, void* stream);
int cretif_gemm_skinny_max_rows(void);

// C[M,N] (= or +=) A[M,K] · W[N,K]^T on the tcgen05 tensor cores (TMA + TMEM), bfloat16
// operands, C bfloat16 or float32 (+= only float32).  bn = 64/128/192/256 picks the tile width,
// 0 lets the launcher choose.  A wait that expires sets bit 2 of *fault.
int cretif_gemm_tc(const void* A, const void* W, void* C, int c_dt, int M, int N, int K, int lda,
                   int ldw, int ldc, int accumulate, int bn, unsigned int* fault, void* stream);

// (For tests that run both.)  Epilogue warps of the tensor-core product: 4 or 8; 0, the default,
// chooses per launch.  Returns the old setting.
int cretif_set_tc_epilogue_warps(int n);

// (For tests that run both.)  Adding into a float32 matrix, and storing the SiLU product,
// through shared memory and TMA: on by default.  Returns the old setting.
int cretif_set_tc_bulk_add(int on);

// (For tests that run both.)  Two CTAs on a tile (cta_group::2) for the float32 add and the
// SiLU product: -1 where the launcher sees fit (default), 0 never, 1 wherever the kernel takes
// the product.  Returns the old setting.
int cretif_set_tc_pair(int mode);

// The same product with fused epilogues (see gemm_tc.cu): SiLU·mul for the stacked gate|up
// matrix whose rows are interleaved in blocks of 64 (I % 64 == 0), and rotary + cache write for
// the stacked q|k|v matrix (head_dim 64 or 128, rotary over the whole head).
int cretif_gemm_tc_silu(const void* A, const void* Wgu, void* act, int M, int I, int K, int lda,
                        int ldw, unsigned int* fault, void* stream);
int cretif_gemm_tc_qkv_rope(const void* A, const void* Wqkv, void* Q, int ldq, const float* cos_t,
                            const float* sin_t, int pairing, int nh, int nkv, int hd,
                            const int* tok_pos, const int* tok_seq, const int* seq_slot,
                            const int* table, int table_stride, void* kc, void* vc, int bt,
                            int write_cache, int M, int K, int lda, int ldw, unsigned int* fault,
                            void* stream);

// Causal grouped-query attention over the block cache, any step shape.
int cretif_attn_simt(const void* q, int ldq, void* out, int ldo, int dt, const void* kc,
                     const void* vc, const int* table, int table_stride, const int* tok_pos,
                     const int* tok_seq, const int* seq_slot, int nh, int nkv, int hd, float scale,
                     int window, int bt, int T, void* stream);

// Decode attention (one query token per sequence), bfloat16, keys split into n_splits <= 64
// ranges per (sequence, kv head); part_o/part_ml are float32 scratch of the sizes that
// cretif_attn_decode_scratch_floats reports, counters is int32 [B * nkv], zero before the
// first launch and left zero by every launch.  block tokens must be 64.
int cretif_attn_decode_scratch_floats(int B, int nh, int hd, int n_splits, long long* part_o,
                                      long long* part_ml);
int cretif_attn_decode(const void* q, int ldq, void* out, int ldo, const void* kc, const void* vc,
                       const int* table, int table_stride, const int* tok_pos, const int* tok_seq,
                       const int* seq_slot, int nh, int nkv, int hd, float scale, int window,
                       int bt, int B, int n_splits, float* part_o, float* part_ml, int* counters,
                       unsigned int* fault, void* stream);

// The same operation on the tensor cores (mma.sync, TMA-swizzled tiles), head_dim <= 128;
// same scratch and counters.  n_blocks is the cache's block count.  With part_o null and at
// most 8 ranges, the ranges of a sequence form a thread-block cluster and are merged through
// distributed shared memory: no scratch, no counters.
int cretif_attn_decode_mma(const void* q, int ldq, void* out, int ldo, const void* kc,
                           const void* vc, long long n_blocks, const int* table, int table_stride,
                           const int* tok_pos, const int* tok_seq, const int* seq_slot, int nh,
                           int nkv, int hd, float scale, int window, int bt, int B, int n_splits,
                           float* part_o, float* part_ml, int* counters, unsigned int* fault,
                           void* stream);

// Fused decode projections (see decode_fused.cu).  H is the float32 residual stream; when it
// is given, x = bf16(rmsnorm(H[rows])) is computed in the kernel, else X (bfloat16) is read.
int cretif_fused_linear(const void* X, int ldx, const float* H, const float* norm_w,
                        const int* rows, float eps, const void* W, int ldw, void* C, int c_dt,
                        int ldc, int accumulate, int M, int N, int K, unsigned int* fault,
                        void* stream);
int cretif_fused_qkv_rope(const float* H, const float* norm_w, float eps, const void* Wqkv, int ldw,
                          void* Q, int ldq, const float* cos_t, const float* sin_t, int pairing,
                          int nh, int nkv, int hd, const int* tok_pos, const int* tok_seq,
                          const int* seq_slot, const int* table, int table_stride, void* kc,
                          void* vc, int bt, int write_cache, int M, int K, unsigned int* fault,
                          void* stream);
int cretif_fused_gate_up_silu(const float* H, const float* norm_w, float eps, const void* Wgu,
                              int ldw, void* act, int I, int gu_block, int M, int K,
                              unsigned int* fault, void* stream);
int cretif_fused_smem_ok(int M, int K, int norm_prologue);
// The three switches below exist so that tests can run both variants of a kernel on one
// shape; an ordinary run never touches them.
// Programmatic dependent launch of the fused kernels on (default) or off; returns the old value.
int cretif_set_dependent_launch(int on);
// Matrices with at least k columns, or of at least min_bytes bytes (negative: unchanged), take
// the shared-memory streaming variant (decode_stream.cuh); returns the old column threshold.
int cretif_set_stream_min_k(int k, long long min_bytes);
long long cretif_stream_min_bytes(void);
// The register variant with more than eight rows and a norm prologue shares the rows'
// normalisation among the CTAs of a thread-block cluster of up to n (1: every CTA norms
// every row itself; at most 4, the default).  Returns the old value; n < 1 leaves it.
int cretif_set_fused_cluster(int n);

// Causal attention for whole prompts on tcgen05 (bfloat16, head_dim a multiple of 16 up to
// 128, 64-token cache blocks).  qkv rows hold the query heads first; sequence b brings the
// tokens cu_seqlens[b] .. cu_seqlens[b+1]-1 at positions seq_start[b] ..; max_new is the
// most tokens one sequence brings.
int cretif_attn_prefill_tc(const void* qkv, int ldq, int T, void* out, int ldo, const void* kc,
                           const void* vc, long long n_blocks, const int* table, int table_stride,
                           const int* cu_seqlens, const int* seq_start, const int* seq_slot,
                           int nh, int nkv, int hd, float scale, int window, int bt, int B,
                           int max_new, unsigned int* fault, void* stream);

// One CTA waits, with the library's bounded wait, on a barrier that nothing completes; after
// `limit` polls (at most 2^20) it gives up, sets bit 2 of *fault and returns.  *polls (may be
// null) receives `limit` when the kernel has run.  Nothing faults or hangs: it exists so that
// the path from an expired wait to the host's error can be exercised.
int cretif_wait_that_expires(unsigned int limit, unsigned int* fault, unsigned int* polls,
                             void* stream);

// (For tests that run all.)  Which kernel cretif_attn_prefill_tc gives head sizes up to 64
// without a window: -1 as the launcher sees fit (default), 0 two threads per row, 1 a thread per
// row and two query tiles per CTA, 2 a thread per row and one tile per CTA.  Returns the old
// setting.
int cretif_set_prefill_pairing(int mode);

// How often variant v of a kernel (cretif::Variant in common.cuh) has been launched; -1 for an
// unknown v.  For tests that must know which path ran.
int cretif_variant_count(int v);

// One token id per row of logits: greedy (temperature <= 0), temperature, or top-k.  The
// kernel reads the seed from *seed_dev when that is not null, else takes `seed`.
int cretif_sample(const float* logits, int ld, int rows, int V, float temperature, int top_k,
                  unsigned long long seed, const unsigned long long* seed_dev,
                  const long long* request, int* draw, int* out, void* stream);
float cretif_uniform01(unsigned long long seed, long long request, int draw);
int cretif_max_top_k(void);

#ifdef __cplusplus
}
#endif
