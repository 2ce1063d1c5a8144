/*
 * fk_b200.h -- C ABI of libfk_b200.so: the decode hot path of the FastKernels
 * nano-vllm-style serving engine as hand-written sm_100a CUDA kernels.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless
 *     its comment says "host";
 *   - strides are in ELEMENTS of the tensor's dtype, sizes in elements unless
 *     the name ends in _bytes;
 *   - the activation / cache dtype is bf16 (2 bytes); accumulation is fp32;
 *   - `stream` is a cudaStream_t (CUstream) passed as an opaque pointer; the
 *     call only enqueues work on it: no allocation, no host synchronisation,
 *     so every call can be captured into a CUDA graph;
 *   - the return value is FK_OK (0) or a negative fk_status code after
 *     host-side argument validation; nothing throws.  fk_last_error() gives
 *     the message of the last failing call on the calling thread;
 *   - kernels never trap: device-side problems (an out-of-range slot or page
 *     id, a wait that ran out) are recorded in the optional `status` word
 *     (one int32 in device memory, 0 = clean) and the offending access is
 *     skipped.
 *
 * Each declaration cites the reference interface it replaces
 * (paths relative to the reference repository root).
 */
#ifndef FK_B200_H_
#define FK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* fk_stream_t; /* cudaStream_t */

enum fk_status {
  FK_OK = 0,
  FK_ERR_INVALID_ARG = -1, /* null pointer, negative size, bad stride        */
  FK_ERR_UNSUPPORTED = -2, /* a shape this build has no kernel for            */
  FK_ERR_WORKSPACE = -3,   /* workspace pointer null or too small             */
  FK_ERR_ALIGNMENT = -4,   /* pointer / stride breaks a 16-byte requirement   */
  FK_ERR_CUDA = -5         /* a CUDA runtime / driver call failed             */
};

/* Device-side status bits written (atomicOr) into the optional status word. */
enum fk_device_status {
  FK_DEV_BAD_SLOT = 1,     /* slot_mapping entry >= num_slots: row skipped    */
  FK_DEV_BAD_PAGE = 2,     /* block_table entry outside [0, num_blocks)       */
  FK_DEV_WAIT_TIMEOUT = 4, /* a bounded mbarrier / flag wait ran out          */
  FK_DEV_BAD_POSITION = 8, /* position outside [0, max_position)              */
  FK_DEV_TMEM_BASE = 16    /* tensor memory was not handed out from column 0  */
};

/* Library version: major*10000 + minor*100 + patch. */
int fk_version(void);

/* Message of the last failing call on this thread ("" if none). Host pointer,
 * valid until the next failing call on the same thread. */
const char* fk_last_error(void);

/* Programmatic dependent launch between the library's kernels (default on; the
 * environment variable FK_B200_PDL=0 turns it off).  Returns the previous
 * setting.  With it on, a kernel's launch latency and prologue overlap the tail
 * of the kernel before it on the same stream; results are identical. */
int fk_set_pdl(int enabled);

/* Number of kernels this library has launched since load (host counter). */
int64_t fk_launch_count(void);

/* ------------------------------------------------------------------------
 * KV-cache store.
 * Replaces StoreKVCache.forward(key, value, k_cache, v_cache, slot_mapping)
 * (fastkernels/tasks/baseline/L1/store_kvcache.py:71-82, kernel 16-35):
 *   for every token i with slot = slot_mapping[i] >= 0:
 *     k_cache.view(-1, row_elems)[slot] = key[i]; same for value.
 * key/value: [num_tokens, row_elems] with row strides key_stride/value_stride
 * (views into a packed qkv buffer are fine); caches: contiguous
 * [num_slots, row_elems].  slot_mapping is int32 (slot_is_int64 == 0) or
 * int64.  Rows with slot < 0 are skipped; rows with slot >= num_slots are
 * skipped and flagged FK_DEV_BAD_SLOT.  Raw 16-bit copy: bit-exact.
 * ---------------------------------------------------------------------- */
int fk_store_kvcache(const void* key, const void* value, void* k_cache,
                     void* v_cache, const void* slot_mapping,
                     int slot_is_int64, int64_t num_tokens, int64_t row_elems,
                     int64_t key_stride, int64_t value_stride,
                     int64_t num_slots, int32_t* status, fk_stream_t stream);

/* HND pool [num_blocks, num_kv_heads, page_size, head_dim].  Replaces
 * StoreKVCacheHND.forward (fastkernels/tasks/baseline/L1/store_kvcache.py:85-101,
 * kernel 38-68): slot -> block = slot / page_size, offset = slot % page_size.
 * key/value: [num_tokens, num_kv_heads, head_dim], heads dense, token strides
 * given.  Same skipping / flagging rules as fk_store_kvcache.  Bit-exact. */
int fk_store_kvcache_hnd(const void* key, const void* value, void* k_cache,
                         void* v_cache, const void* slot_mapping,
                         int slot_is_int64, int64_t num_tokens, int num_kv_heads,
                         int head_dim, int64_t key_stride, int64_t value_stride,
                         int page_size, int64_t num_blocks, int32_t* status,
                         fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Paged GQA decode attention (one query token per sequence).
 * Replaces FlashAttnDecode.forward(q, k_cache, v_cache, cache_seqlens,
 *   block_table=..., softmax_scale=..., causal=True, max_seq_len=...)
 * (fastkernels/tasks/baseline/L1/flash_attn_decode.py:113-181); same maths as
 * Attention._decode_torch (fastkernels/tasks/baseline/L2/attention_impl.py:
 * 598-664): out[i,h] = softmax(scale * q[i,h] . K_i[:L_i, h/g]^T) V_i[:L_i, h/g]
 * with K_i/V_i gathered through block_tables[i, p]*block_size + offset.
 *
 * q:   [batch, num_q_heads, head_dim], token stride q_stride_token, heads
 *      contiguous (stride head_dim).  out likewise with out_stride_token.
 * k_cache/v_cache: paged pool, contiguous within a block, blocks
 *      kv_block_stride elements apart; kv_layout 0 = NHD
 *      [num_blocks, block_size, num_kv_heads, head_dim] (the flash-attn path),
 *      kv_layout 1 = HND [num_blocks, num_kv_heads, block_size, head_dim] (what
 *      TRTLLMDecode reads, fastkernels/tasks/baseline/L1/flashinfer_decode.py:
 *      44-107, the reference's default on B200 with page size 16).
 * context_lens: [batch] int32 (0 = padded row: output row is zero-filled).
 * block_tables: [batch, >= ceil(L/block_size)] int32, rows
 *      block_table_stride apart (may exceed the live column count).
 * max_splits: upper bound on KV splits per sequence the workspace was sized
 *      for (fk_paged_decode_attn_workspace_bytes).  The split size is chosen
 *      on the device from context_lens, so one captured launch serves every
 *      replay.
 * Supported: head_dim 128, block_size 16, 32 or a multiple of 64,
 * num_q_heads/num_kv_heads in {1,2,4,8,16}, bf16.
 * Launches: plan + main + merge kernel; a small call (batch * num_kv_heads <= SM
 *      count and block tables of at most 2048 tokens) is a single launch in which
 *      every (sequence, KV head) pair has its own CTA and nothing is split.
 * ---------------------------------------------------------------------- */
size_t fk_paged_decode_attn_workspace_bytes(int batch, int num_q_heads,
                                            int head_dim, int max_splits);

int fk_paged_decode_attn(const void* q, int64_t q_stride_token, void* out,
                         int64_t out_stride_token, const void* k_cache,
                         const void* v_cache, int64_t num_blocks,
                         int block_size, int64_t kv_block_stride, int kv_layout,
                         const int32_t* context_lens,
                         const int32_t* block_tables,
                         int64_t block_table_stride, int batch,
                         int num_q_heads, int num_kv_heads, int head_dim,
                         float softmax_scale, int max_splits, void* workspace,
                         size_t workspace_bytes, int32_t* status,
                         fk_stream_t stream);

/* The split schedule depends only on context_lens, which every layer of a decode
 * step shares (the engine sets one Context per step,
 * fastkernels/infra/engine.py:6057-6063).  fk_paged_decode_attn_plan computes it
 * once into the workspace; fk_paged_decode_attn_planned is fk_paged_decode_attn
 * without the plan launch and may be called for any number of layers afterwards
 * with the same workspace, context_lens, block_tables, batch, head counts and
 * max_splits (each call leaves the schedule ready for the next). */
int fk_paged_decode_attn_plan(const int32_t* context_lens,
                              const int32_t* block_tables,
                              int64_t block_table_stride, int block_size, int batch,
                              int num_q_heads, int num_kv_heads, int head_dim,
                              int max_splits, void* workspace,
                              size_t workspace_bytes, int32_t* status,
                              fk_stream_t stream);

int fk_paged_decode_attn_planned(const void* q, int64_t q_stride_token, void* out,
                                 int64_t out_stride_token, const void* k_cache,
                                 const void* v_cache, int64_t num_blocks,
                                 int block_size, int64_t kv_block_stride,
                                 int kv_layout,
                                 const int32_t* context_lens,
                                 const int32_t* block_tables,
                                 int64_t block_table_stride, int batch,
                                 int num_q_heads, int num_kv_heads, int head_dim,
                                 float softmax_scale, int max_splits,
                                 void* workspace, size_t workspace_bytes,
                                 int32_t* status, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * RMSNorm and fused residual-add + RMSNorm.
 * Replace RMSNorm.forward(x, residual=None)
 * (fastkernels/tasks/baseline/L1/rms_norm.py:153-164; kernels
 * fastkernels/tasks/baseline/L1/rms_norm.cu:1251-1336 and 1342-1410):
 *   fk_rmsnorm:  out = bf16(float(x) * rsqrt(mean(x^2)+eps) * float(w))
 *     rows of `cols` elements; x rows x_stride apart (per-head q/k norm on a
 *     strided [N, H, D] view passes rows = N*H with the 3-D form below);
 *   fk_fused_add_rmsnorm (in place, both tensors):
 *     residual = bf16(x + residual); x = bf16(float(residual) * rsqrt(...) * w)
 * ---------------------------------------------------------------------- */
int fk_rmsnorm(const void* x, int64_t x_stride_outer, int64_t x_stride_inner,
               int64_t inner, void* out, int64_t out_stride_outer,
               int64_t out_stride_inner, const void* weight, float eps,
               int64_t outer, int64_t cols, fk_stream_t stream);

int fk_fused_add_rmsnorm(void* x, int64_t x_stride, void* residual,
                         int64_t residual_stride, const void* weight,
                         float eps, int64_t rows, int64_t cols,
                         fk_stream_t stream);

/* ------------------------------------------------------------------------
 * NeoX rotary embedding, in place on query and key.
 * Replaces RotaryEmbedding.forward(positions, query, key)
 * (fastkernels/tasks/baseline/L1/rotary_emb.py:179-191; kernel
 * fastkernels/tasks/baseline/L1/rotary_emb.cu:332-423):
 *   (x_i, x_{i+D/2}) <- (x_i c - x_{i+D/2} s, x_{i+D/2} c + x_i s),
 *   c,s = cache[pos, i], cache[pos, D/2+i] rounded to bf16, fp32 maths, one
 *   rounding.  cos_sin_cache: [max_position, head_dim], fp32
 *   (cache_is_fp32 = 1; rounded to bf16 in the kernel, as the reference's
 *   per-call cast does) or bf16.  positions: [num_tokens] int64.
 * ---------------------------------------------------------------------- */
int fk_rope_neox(const int64_t* positions, void* query, int64_t q_stride,
                 int num_q_heads, void* key, int64_t k_stride,
                 int num_kv_heads, int head_dim, const void* cos_sin_cache,
                 int cache_is_fp32, int64_t max_position, int64_t num_tokens,
                 int32_t* status, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Fused QKV split + optional per-head q/k RMSNorm + NeoX RoPE + KV store.
 * Replaces, in one pass over the packed projection output, the chain in
 * LlamaAttention.forward (fastkernels/tasks/baseline/L2/attention.py:113-156):
 *   qkv.split -> [q_norm/k_norm] -> rotary_emb -> Attention.forward_impl's
 *   StoreKVCache (fastkernels/tasks/baseline/L2/attention_impl.py:313-325).
 * qkv: [num_tokens, (Hq + 2 Hkv) * D] with row stride qkv_stride; q and k are
 * rotated IN PLACE inside qkv (so a later reader of the q view sees the same
 * values the reference produces); rotated k and raw v are also written to
 * k_cache/v_cache at slot_mapping[i] (int32; < 0 skips the store).
 * kv_layout 0 = NHD cache (block_size unused), 1 = HND cache with pages of
 * block_size tokens.
 * q_norm_weight / k_norm_weight: [D] bf16 or NULL (no per-head norm).
 * Rounding points match the unfused chain: normed value rounded to bf16, then
 * rotated in fp32 and rounded once.
 * ---------------------------------------------------------------------- */
int fk_qkv_rope_store(void* qkv, int64_t qkv_stride, int num_q_heads,
                      int num_kv_heads, int head_dim,
                      const int64_t* positions, const void* cos_sin_cache,
                      int cache_is_fp32, int64_t max_position,
                      const void* q_norm_weight, const void* k_norm_weight,
                      float norm_eps, void* k_cache, void* v_cache,
                      const int32_t* slot_mapping, int64_t num_slots,
                      int block_size, int kv_layout, int64_t num_tokens,
                      int32_t* status, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * SiLU-and-multiply.  Replaces SiluAndMul.forward(x)
 * (fastkernels/tasks/baseline/L1/silu_and_mul.py:32-35; kernel
 * fastkernels/tasks/baseline/L1/silu_and_mul.cu:715-740):
 *   out[t, j] = bf16(float(bf16(silu(x[t, j]))) * float(x[t, d + j]))
 * x: [rows, 2*d] row stride x_stride; out: [rows, d] row stride out_stride.
 * ---------------------------------------------------------------------- */
int fk_silu_and_mul(const void* x, int64_t x_stride, void* out,
                    int64_t out_stride, int64_t rows, int64_t d,
                    fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Dense projection y = x W^T (+ bias): bf16 x bf16 -> fp32 (TMEM) -> bf16.
 * Replaces Matmul.forward(input, weight, bias)
 * (fastkernels/tasks/baseline/L1/linear.py:13-17) and the F.linear calls of
 * {QKV,MergedColumn,Column,Row}ParallelLinear.forward
 * (fastkernels/tasks/baseline/L2/parallel_linear.py:78-81,157-160,237-240,
 * 327-335).  x: [m, k] row stride x_stride; w: [n, k] row-major contiguous
 * (the nn.Linear layout); y: [m, n] row stride y_stride; bias [n] or NULL.
 * k % 64 == 0, n % 8 == 0.  m <= 256 (decode) runs the weight-streaming kernel;
 * m > 256 (prefill) runs a 256 x 256 tile kernel, needs no workspace
 * (fk_gemm_bf16_workspace_bytes returns 0) and 16-byte aligned rows of y.
 * workspace: fk_gemm_bf16_workspace_bytes(m, n, k) bytes, 256-byte aligned,
 * ZERO-INITIALISED once by the caller (cudaMemset) before its first use: it holds
 * the stream-K flags and fp32 partial tiles, and every call leaves it zeroed
 * again, so one buffer can serve all GEMMs issued on one stream.  Two calls that
 * may run concurrently need separate workspaces.
 * After FK_DEV_WAIT_TIMEOUT was reported in `status` the results of that call are
 * undefined and a late contributor may have left a flag raised: zero the first
 * 1024 bytes of the workspace again (stream-ordered) before the next call.
 * ---------------------------------------------------------------------- */
size_t fk_gemm_bf16_workspace_bytes(int64_t m, int64_t n, int64_t k);

int fk_gemm_bf16(const void* x, int64_t x_stride, const void* w,
                 const void* bias, void* y, int64_t y_stride, int64_t m,
                 int64_t n, int64_t k, void* workspace,
                 size_t workspace_bytes, int32_t* status, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Gate/up projection fused with SiLU-and-multiply: y = silu(x Wg^T) * (x Wu^T)
 * with W = [Wg; Wu] the merged [n, k] matrix (n/2 gate rows, then n/2 up rows).
 * Replaces the pair MergedColumnParallelLinear.forward
 *   (fastkernels/tasks/baseline/L2/parallel_linear.py:157-160) + SiluAndMul.forward
 *   (fastkernels/tasks/baseline/L1/silu_and_mul.py:32-35) as LlamaMLP.forward
 *   chains them (fastkernels/tasks/baseline/L2/llama_mlp.py:35-38).
 * Rounding points are those of the two separate ops: both projection outputs are
 * rounded to bf16 (+ bias, [n] or null), silu(gate) is rounded to bf16, the
 * product once more.  y is [m, n/2] bf16; the [m, n] intermediate never exists.
 * Same workspace as fk_gemm_bf16(m, n, k).  Only shapes that take the persistent
 * stream-K schedule have this single-launch form (m <= 256, n % 128 == 0, more
 * weight tiles than half the SMs): fk_gemm_bf16_silu_mul_fusable says which;
 * other shapes return FK_ERR_UNSUPPORTED and the caller runs the two ops.
 * ---------------------------------------------------------------------- */
int fk_gemm_bf16_silu_mul_fusable(int64_t m, int64_t n, int64_t k);
int fk_gemm_bf16_silu_mul(const void* x, int64_t x_stride, const void* w,
                          const void* bias, void* y, int64_t y_stride, int64_t m,
                          int64_t n, int64_t k, void* workspace,
                          size_t workspace_bytes, int32_t* status, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Persistent decode block: the kernels a decoder layer runs between two
 * attention calls, as ONE launch (one persistent CTA per SM) that walks a
 * program of up to 8 phases.  It computes what the reference computes with
 *   RowParallelLinear.forward (o_proj)     fastkernels/tasks/baseline/L2/parallel_linear.py:327-335
 *   RMSNorm.forward(x, residual)            fastkernels/tasks/baseline/L1/rms_norm.py:153-164
 *   LlamaMLP.forward                        fastkernels/tasks/baseline/L2/llama_mlp.py:35-38
 *   LlamaDecoderLayer.forward (norm order)  fastkernels/tasks/baseline/L3/llama_decoder.py:34-42
 *   LlamaAttention.forward up to the attention call (qkv_proj, q/k norm, RoPE)
 *                                           fastkernels/tasks/baseline/L2/attention.py:113-150
 *   StoreKVCache.forward                    fastkernels/tasks/baseline/L1/store_kvcache.py:71-82
 * with the rounding points of the separate entry points above (fk_gemm_bf16,
 * fk_gemm_bf16_silu_mul, fk_fused_add_rmsnorm / fk_rmsnorm, fk_qkv_rope_store).
 * Phases run in order; each sees everything the earlier ones wrote (a grid-wide
 * barrier with bounded waits -> FK_DEV_WAIT_TIMEOUT), while the weight tiles of
 * later projections are already being fetched.  Phase kinds and the fields read:
 *   FK_PHASE_GEMM            y[m, n] = x[m, k] w[n, k]^T (+ bias[n])
 *   FK_PHASE_GEMM_SILU_MUL   y[m, n/2] = silu(x wg^T) * (x wu^T), w = [wg; wu], n % 128 == 0
 *       x, x_stride, w, bias, y, y_stride, n, k              (k % 64 == 0)
 *   FK_PHASE_ADD_RMSNORM     residual = bf16(x + residual) (x null: nothing added);
 *                            y = rmsnorm(residual) * norm_weight over n columns
 *       x, x_stride, residual, residual_stride, norm_weight, eps, y, y_stride, n
 *   FK_PHASE_QKV_ROPE_STORE  fk_qkv_rope_store on x = packed qkv rows (head_dim 128,
 *                            bf16 cos/sin cache), at most once per launch
 *       x, x_stride, num_q_heads, num_kv_heads, head_dim, positions, cos_sin_cache,
 *       cache_is_fp32 (must be 0), max_position, q_norm_weight, k_norm_weight, eps,
 *       k_cache, v_cache, slot_mapping, num_slots, block_size, kv_layout
 * m <= 128 rows, at most 4 projections per launch.  workspace: fk_decode_block_
 * workspace_bytes(m) bytes, 256-byte aligned, zero-initialised once; a launch
 * leaves it zeroed (unless a wait timed out: re-zero it then).  Launches that
 * share a workspace must not overlap on the GPU.  Every CTA must be resident for
 * the barriers to complete: the grid is one CTA per SM, so give the kernel the
 * whole device (no other long-running kernel alongside).
 * ---------------------------------------------------------------------- */
enum fk_block_phase_kind {
  FK_PHASE_GEMM = 1,
  FK_PHASE_GEMM_SILU_MUL = 2,
  FK_PHASE_ADD_RMSNORM = 3,
  FK_PHASE_QKV_ROPE_STORE = 4
};
typedef struct fk_block_phase {
  int32_t kind;
  const void* x; int64_t x_stride;
  const void* w; const void* bias;
  void* y; int64_t y_stride;
  int64_t n, k;
  void* residual; int64_t residual_stride;
  const void* norm_weight; float eps;
  int32_t num_q_heads, num_kv_heads, head_dim;
  const int64_t* positions;
  const void* cos_sin_cache; int32_t cache_is_fp32; int64_t max_position;
  const void* q_norm_weight; const void* k_norm_weight;
  void* k_cache; void* v_cache;
  const int32_t* slot_mapping; int64_t num_slots;
  int32_t block_size, kv_layout;
} fk_block_phase;
size_t fk_decode_block_workspace_bytes(int64_t m);
int fk_decode_block(const fk_block_phase* phases, int num_phases, int64_t m,
                    void* workspace, size_t workspace_bytes, int32_t* status,
                    fk_stream_t stream);

/* ------------------------------------------------------------------------
 * fk_gemm_bf16 for callers that cannot allocate device memory.
 * No counterpart in the reference: this entry point exists for hosts that get
 * their tensors from someone else and may not call cudaMalloc themselves -- a
 * plugin running inside another runtime's memory pool, code on a stream that is
 * being captured, a sandbox whose allocator is off limits.  Same arguments and
 * results as fk_gemm_bf16 minus the workspace: the stream-K scratch is a
 * ~5 MiB array built into the library image (each GPU that loads the library
 * keeps it until the process exits).
 *   - limit: m <= 64 (the scratch is sized for it); a larger m returns
 *     FK_ERR_UNSUPPORTED and says so in fk_last_error();
 *   - the call itself allocates nothing: no cudaMalloc / cudaFree, no allocating
 *     library routine;
 *   - the FIRST call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); the device the stream belongs to must be the
 *     current device.  Make that first call before any stream capture begins: a
 *     first call on a stream that is being captured returns FK_ERR_UNSUPPORTED.
 *     The flag words need no clearing at set-up: the array is zero when the
 *     library is loaded;
 *   - every call shares the one array, which keeps the previous call's partial
 *     tiles (only the flag words need to be zero, and each call leaves them
 *     zero): calls that overlap on the GPU -- two streams, two host threads --
 *     race on it; issue them on one stream, or use fk_gemm_bf16 with separate
 *     workspaces.
 * ---------------------------------------------------------------------- */
int fk_gemm_bf16_static(const void* x, int64_t x_stride, const void* w,
                        const void* bias, void* y, int64_t y_stride, int64_t m,
                        int64_t n, int64_t k, int32_t* status,
                        fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Greedy sampling over the lm-head logits: per row the maximum (as fp32) and
 * its index.  Replaces lm_logits[:bs].max(dim=-1) in the captured decode graph
 * (fastkernels/infra/engine.py:6994-6996).  Ties go to the LOWEST index; NaN
 * never wins.  x: [rows, cols] bf16 row stride x_stride; out_val [rows] fp32
 * (may be NULL); out_idx [rows] int64.
 * ---------------------------------------------------------------------- */
int fk_argmax_bf16(const void* x, int64_t x_stride, int64_t rows, int64_t cols,
                   float* out_val, int64_t* out_idx, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Tensor-parallel all-reduce fused with residual add + RMSNorm, over peer memory.
 * Replaces AllReduce.forward (fastkernels/tasks/baseline/L1/allreduce.py:37-55,
 * one-shot kernel fastkernels/tasks/baseline/L1/allreduce.cu:193-212) followed by
 * RMSNorm.forward(x, residual) (fastkernels/tasks/baseline/L1/rms_norm.py:153-164);
 * the reference's own fused form is
 * fastkernels/tasks/baseline/L2/flashinfer_allreduce_fusion.py:227-297.
 *
 * Communication buffer (one per rank, same size on all ranks):
 *   fk_comm_alloc        cudaMalloc + zero; layout = fk_comm_header_bytes() of flag
 *                        words, then caller-defined data slots
 *   fk_comm_ipc_export   64-byte CUDA IPC handle of the buffer (send to the peers)
 *   fk_comm_ipc_import   map a peer's buffer, returns its local address
 * These four are set-up calls (they allocate / map; not for use during capture).
 *
 * fk_allreduce_add_rmsnorm: bases = HOST array of nranks device addresses, entry r
 * being rank r's buffer as mapped in this process (bases[rank] is the local one).
 * Each rank's partial [rows, cols] bf16 (rows dense) sits at bases[r] +
 * slot_offset_bytes.  Computes, identically on every rank,
 *   s = bf16(sum_r y_r) (fp32, rank order); residual = bf16(s + residual) in place;
 *   out = bf16(float(residual) * rsqrt(mean(residual^2) + eps) * float(weight)).
 * Callers alternate between (at least) two slots on consecutive calls; all ranks
 * must issue the same sequence of calls.  rows <= 512, cols % 8 == 0, <= 16384.
 * Waits on peers are bounded (2 s) and reported as FK_DEV_WAIT_TIMEOUT.
 *
 * fk_allreduce_add_rmsnorm_staged: the same result (bit for bit) through a
 * two-stage exchange, for payloads where pulling every rank's rows costs more
 * than a second flag round -- the regime in which the reference switches from its
 * one-stage to its two-stage kernel
 * (fastkernels/tasks/baseline/L1/allreduce.cu:214-250, switch-over 404-415).
 * fk_allreduce_two_stage_preferred is this build's own switch-over, set from
 * measurements on B200: one stage at every decode payload, two from 4 MiB on 8 ranks.  Row i is reduced by rank
 * i % nranks alone, which pushes the bf16 sum into rows*cols*2 bytes of staging at
 * bases[r] + staging_offset_bytes of every peer r; the staging rows must not
 * overlap the data slot, and calls alternate between two staging areas exactly as
 * they alternate between two slots.  Calls of both kinds may be mixed freely as
 * long as all ranks issue the same sequence.
 *
 * Pushed exchange (the projection and the collective as one kernel):
 * fk_gemm_bf16_push is fk_gemm_bf16 for a row-parallel projection
 * (RowParallelLinear.forward, fastkernels/tasks/baseline/L2/parallel_linear.py:
 * 327-335) whose result is all-reduced next: instead of y, every tile's epilogue
 * stores its outputs straight into the receive areas of ALL ranks over NVLink, as
 * 8-byte {two bf16, call number} words, each written atomically -- the transfer
 * runs tile by tile under the rest of the projection.  dst = HOST array of nranks
 * device addresses, entry r = THIS sender's area inside rank r's buffer
 * ([m][n / 2] words, 16-byte aligned); call_counters = the per-row counters in this
 * rank's own header (buffer + fk_comm_epoch_offset()).
 * fk_allreduce_add_rmsnorm_pushed then reads only local memory: per element it
 * waits (bounded, 2 s) until the nranks senders' words carry this call's number,
 * sums them in rank order and finishes exactly like fk_allreduce_add_rmsnorm (same
 * bits).  One NVLink traversal per call instead of three, at twice the bytes on
 * the wire: fk_allreduce_push_preferred says where that pays (this build: while
 * (nranks - 1) * rows * cols * 4 <= 4 MiB).  Receive areas of one slot lie
 * sender_stride_bytes apart from ll_offset_bytes on; two slots alternate as above.
 *
 * fk_allreduce_add_rmsnorm_group: all nranks ranks in ONE cooperative launch, for
 * a process that holds every rank's buffer on a single device (a test on one GPU,
 * a host emulating shards).  residuals / outs are HOST arrays of nranks device
 * pointers; staging_offset_bytes = 0 selects the one-stage exchange.  Kernels that
 * wait for one another must not be issued as separate launches on one GPU
 * (nothing guarantees they are resident together); the blocks of a cooperative
 * launch are, and the grid is sized to fit (a block walks several rows when
 * rows * nranks exceeds what the device holds at once).  No counterpart in the
 * reference.
 * ---------------------------------------------------------------------- */
size_t fk_comm_header_bytes(void);
int fk_comm_alloc(size_t bytes, void** ptr);
int fk_comm_free(void* ptr);
int fk_comm_ipc_export(void* ptr, void* handle64);
int fk_comm_ipc_import(const void* handle64, void** peer_ptr);
int fk_comm_ipc_close(void* peer_ptr);
int fk_allreduce_add_rmsnorm(void* const* bases, int nranks, int rank,
                             size_t slot_offset_bytes, void* residual,
                             int64_t residual_stride, const void* weight,
                             float eps, void* out, int64_t out_stride,
                             int64_t rows, int64_t cols, int32_t* status,
                             fk_stream_t stream);
int fk_allreduce_two_stage_preferred(int nranks, int64_t rows, int64_t cols);
size_t fk_comm_epoch_offset(void);
int fk_allreduce_push_preferred(int nranks, int64_t rows, int64_t cols);
int fk_gemm_bf16_push(const void* x, int64_t x_stride, const void* w, const void* bias,
                      int64_t m, int64_t n, int64_t k, void* workspace,
                      size_t workspace_bytes, void* const* dst, int nranks,
                      const void* call_counters, int32_t* status, fk_stream_t stream);
int fk_allreduce_add_rmsnorm_pushed(void* base, int nranks, size_t ll_offset_bytes,
                                    size_t sender_stride_bytes, void* residual,
                                    int64_t residual_stride, const void* weight, float eps,
                                    void* out, int64_t out_stride, int64_t rows, int64_t cols,
                                    int32_t* status, fk_stream_t stream);
int fk_allreduce_add_rmsnorm_staged(void* const* bases, int nranks, int rank,
                                    size_t slot_offset_bytes, size_t staging_offset_bytes,
                                    void* residual, int64_t residual_stride,
                                    const void* weight, float eps, void* out,
                                    int64_t out_stride, int64_t rows, int64_t cols,
                                    int32_t* status, fk_stream_t stream);
int fk_allreduce_add_rmsnorm_group(void* const* bases, int nranks,
                                   size_t slot_offset_bytes, size_t staging_offset_bytes,
                                   void* const* residuals, int64_t residual_stride,
                                   const void* weight, float eps, void* const* outs,
                                   int64_t out_stride, int64_t rows, int64_t cols,
                                   int32_t* status, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Fill `count` 32-bit words at dst (16-byte aligned) with `value`: zeroing of
 * workspaces and KV pools on the caller's stream, and the L2 flush of the
 * micro-benchmarks.  No counterpart in the reference (torch.zeros there).
 * ---------------------------------------------------------------------- */
int fk_fill_u32(void* dst, int64_t count, uint32_t value, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * *out ^= XOR of the `count` 32-bit words at src (16-byte aligned, count a
 * multiple of 4; the caller zeroes *out first): a checksum of a workspace or a
 * KV pool on the caller's stream, and the read-only stream the micro-benchmarks
 * time as the read peak of the device.  No counterpart in the reference.
 * ---------------------------------------------------------------------- */
int fk_xor_u32(const void* src, int64_t count, uint32_t* out, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Variable-length prefill attention, the step before decode.
 * Replaces FlashAttnPrefill.forward
 *   (fastkernels/tasks/baseline/L1/flash_attn_prefill.py:28-74; PyTorch
 *   statement Attention._prefill_torch_from_tensors / _prefill_torch_from_cache,
 *   fastkernels/tasks/baseline/L2/attention_impl.py:624-652).
 * For sequence i, query token t (0-based inside the sequence) and head h:
 *   out = softmax(scale * q . K[i, :n]^T) V[i, :n],  n = k_len_i - q_len_i + t + 1
 * when causal (bottom-right aligned, as flash_attn_varlen_func), n = k_len_i
 * otherwise; q_len_i = cu_seqlens_q[i+1] - cu_seqlens_q[i], k_len_i likewise.
 *   q, out   [total_q, Hq, 128] bf16 with token strides (elements)
 *   out_lse  optional fp32 [Hq, total_q]: natural-log sum of exp of the scaled
 *            scores (-inf for a row without visible keys)
 *   K / V    num_blocks == 0: dense [total_k, Hkv, 128], kv_stride = token stride,
 *            sequence i at rows cu_seqlens_k[i] ..;
 *            num_blocks  > 0: the paged pool as in fk_paged_decode_attn
 *            (kv_stride = block stride, block_size, kv_layout), sequence i's
 *            pages in block_tables[i, :]; only the DIFFERENCES of cu_seqlens_k
 *            are used then (flash_attn_prefill.py:41-42)
 *   cu_seqlens_q, cu_seqlens_k  int32 [num_seqs + 1], on the device
 *   max_seqlen_q  upper bound of q_len_i (sizes the grid)
 * head_dim must be 128.  status: optional device word (FK_DEV_BAD_PAGE,
 * FK_DEV_WAIT_TIMEOUT).
 * ---------------------------------------------------------------------- */
int fk_prefill_attn(const void* q, int64_t q_stride_token, void* out,
                    int64_t out_stride_token, float* out_lse, const void* k,
                    const void* v, int64_t kv_stride, int64_t num_blocks,
                    int block_size, int kv_layout, const int32_t* cu_seqlens_q,
                    const int32_t* cu_seqlens_k, const int32_t* block_tables,
                    int64_t block_table_stride, int num_seqs, int64_t total_q,
                    int64_t total_k, int max_seqlen_q, int num_q_heads,
                    int num_kv_heads, int head_dim, float softmax_scale, int causal,
                    int32_t* status, fk_stream_t stream);

/* ------------------------------------------------------------------------
 * Merge of two partial attention results over disjoint key ranges.
 * Replaces merge_attn_states / MergeAttnStates.forward
 *   (fastkernels/tasks/baseline/L1/merge_attn_states.py:32-122, kernel
 *   merge_attn_states.cu:2440-2580).
 *   out[t,h,:] = (e^{pl} prefix[t,h,:] + e^{sl} suffix[t,h,:]) / (e^{pl} + e^{sl}),
 *   out_lse[h,t] = log(e^{pl} + e^{sl}),  pl = prefix_lse[h,t], sl = suffix_lse[h,t]
 * computed against max(pl, sl) in fp32, one rounding to bf16.  An lse of +inf
 * counts as -inf; when both are -inf the prefix row is passed through and
 * out_lse = -inf.  Tokens t >= prefill_tokens_with_context (negative = all
 * tokens have context) copy the suffix row and suffix lse.
 *   outputs  [num_tokens, num_heads, head_dim] bf16, token and head strides in
 *            elements; lse fp32 [num_heads, num_tokens]; out_lse optional.
 * ---------------------------------------------------------------------- */
int fk_merge_attn_states(void* out, int64_t out_stride_token, int64_t out_stride_head,
                         float* out_lse, const void* prefix_out,
                         int64_t prefix_stride_token, int64_t prefix_stride_head,
                         const float* prefix_lse, const void* suffix_out,
                         int64_t suffix_stride_token, int64_t suffix_stride_head,
                         const float* suffix_lse, int64_t num_tokens, int num_heads,
                         int head_dim, int64_t prefill_tokens_with_context,
                         fk_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* FK_B200_H_ */
