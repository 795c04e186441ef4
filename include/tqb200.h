/*
 * tqb200.h -- C ABI of libtqb200.so, the sm_100a (B200) implementation of the TurboQuant hot path.
 *
 * Every entry point takes raw DEVICE pointers (unless a parameter says "host"), explicit sizes and
 * a CUDA stream (cudaStream_t passed as void*; NULL = the legacy default stream).  The caller
 * allocates every output and every workspace; nothing here allocates device memory.  All calls
 * are stream-ordered and asynchronous; none synchronises.  Return value: 0 on success, a negative
 * TQB_ERR_* code otherwise, with a human-readable message available from tqb_last_error()
 * (thread-local).  No exception crosses this boundary.
 *
 * Each declaration cites the interface of the upstream project (ansschh/turboquant-kv, paths
 * relative to that repository) that it replaces.
 *
 * Conventions shared by all entry points (upstream turboquant_kv/reference.py):
 *   - forward rotation  y = unit @ R^T  (y_j = sum_k unit_k R[j][k], reference.py:301);
 *     inverse rotation  x = y @ R       (reference.py:362);  R is (dim, dim) float32, row-major;
 *   - code = number of boundaries strictly below y (torch.searchsorted, left; reference.py:311);
 *   - a packed row is `bits` planes of ceil(dim/8) bytes, plane i holds bit i of every code,
 *     dimension 8m+t sits at bit 7-t of byte m, padding bits are zero (reference.py:191-224);
 *     packed_dim = bits * ceil(dim/8).
 */
#ifndef TQB200_H_
#define TQB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQB_OK 0
#define TQB_ERR_INVALID (-1)     /* bad argument (shape, bit width, null pointer, alignment) */
#define TQB_ERR_UNSUPPORTED (-2) /* valid upstream, outside what this build implements */
#define TQB_ERR_CUDA (-3)        /* a CUDA runtime call failed; message carries its text */
#define TQB_ERR_WORKSPACE (-4)   /* workspace smaller than tqb_*_workspace_bytes() */

/* element type of floating-point inputs */
#define TQB_F32 0
#define TQB_F16 1
#define TQB_BF16 2

/* ABI version of this header (bumped on any signature change). */
int tqb_abi_version(void);
/* Message of the last failing call on this thread ("" if none). */
const char* tqb_last_error(void);
/* Number of kernels launched by this library in this process (all threads), for accounting. */
int64_t tqb_launch_count(void);

/*
 * Where quantised rows are written.  Input rows are numbered r = a * inner + b (0 <= b < inner).
 *   dense / cache mode (slots == NULL):
 *       out_row = a * stride_a + b * stride_b + offset + (pos ? pos[a / pos_div] : 0)
 *   paged mode (slots != NULL): a = token, b = kv head (inner = kv_heads);
 *       out_row = ((slots[a] / block_size) * inner + b) * block_size + slots[a] % block_size
 *       tokens with slots[a] < 0 are skipped.
 * A plain (n, packed_dim) output is {inner = 1, stride_a = 1, stride_b = 0, offset = 0}.
 */
typedef struct tqb_rowmap {
    int64_t inner;
    int64_t stride_a;
    int64_t stride_b;
    int64_t offset;
    const int32_t* pos; /* device, optional */
    int64_t pos_div;
    const int64_t* slots; /* device, optional */
    int32_t block_size;
} tqb_rowmap;

/* ---- bit-plane pack / unpack ------------------------------------------------------------
 * Replaces torch.ops.turboquant.pack_codes / unpack_codes (csrc/registration.cpp:98-99,
 * csrc/cuda/quant_pack.cu:52-81,117-148) and reference.py:191-255.
 * codes (n, dim) uint8 <-> packed (n, bits*ceil(dim/8)) uint8; bits in 1..8, any dim >= 1. */
int tqb_pack_codes(const uint8_t* codes, int64_t n, int dim, int bits, uint8_t* packed, void* stream);
int tqb_unpack_codes(const uint8_t* packed, int64_t n, int dim, int bits, uint8_t* codes, void* stream);

/* ---- Algorithm 1: quantize / dequantize ---------------------------------------------------
 * Replaces reference.quantize_mse (reference.py:263-317), torch.ops.turboquant.rotate_and_quantize
 * (csrc/registration.cpp:85-88, csrc/cuda/rotate_fused.cu:140-190) and
 * turboquant::quantize_vectors (csrc/core/turboquant_core.cpp:277-343).
 * x: (n, dim) rows of `dtype`, consecutive rows x_stride elements apart; arithmetic in float32.
 * packed / norms are addressed through `map` (NULL = dense); packed rows are packed_dim bytes
 * apart.  bits in 1..4, dim in 8..256 and a multiple of 8. */
int tqb_quantize_mse(const void* x, int dtype, int64_t n, int dim, int64_t x_stride,
                     const float* rotation, const float* boundaries, int bits, uint8_t* packed,
                     float* norms, const tqb_rowmap* map, void* stream);

/* Replaces reference.dequantize_mse (reference.py:320-367) and turboquant::dequantize_vectors
 * (csrc/core/turboquant_core.cpp:345-401).  out: (n, dim) of out_dtype. */
/* Large calls (dim 64 / 128, 2-4 bits, at least 512 rows, 16-byte aligned rows) run on the tensor cores
 * (csrc/quantize_tc.cu: tcgen05.mma with bf16 operand splits, exact re-quantisation of rows near a decision
 * boundary), with the same codes and norms as the FFMA kernel.  Its waits are bounded; tqb_quantize_status
 * reads and clears the error word one of them would raise (0 = all good; non-zero = the outputs of the
 * quantise calls since the last query are not to be trusted).  Synchronises `stream`.  No upstream counterpart. */
int tqb_quantize_status(void* stream);
int tqb_dequantize_mse(const uint8_t* packed, const float* norms, int64_t n, int dim,
                       const float* rotation, const float* centroids, int bits, void* out,
                       int out_dtype, void* stream);

/* ---- Algorithm 2: quantize / dequantize with the 1-bit QJL residual ------------------------
 * Replaces reference.quantize_prod (reference.py:392-469).  `boundaries`/`centroids` are the
 * (bits-1)-bit codebook, `qjl` the (dim, dim) Gaussian matrix S, `qjl_rot` = S @ R^T (dim, dim)
 * precomputed by the caller.  Outputs (dense): mse_packed (n, (bits-1)*ceil(dim/8)), signs
 * (n, ceil(dim/8)), res_norms (n), norms (n).  bits in 2..5. */
int tqb_quantize_prod(const void* x, int dtype, int64_t n, int dim, int64_t x_stride,
                      const float* rotation, const float* boundaries, const float* centroids,
                      const float* qjl_rot, int bits, uint8_t* mse_packed, uint8_t* signs,
                      float* res_norms, float* norms, void* stream);

/* Replaces reference.dequantize_prod (reference.py:472-533). */
int tqb_dequantize_prod(const uint8_t* mse_packed, const uint8_t* signs, const float* res_norms,
                        const float* norms, int64_t n, int dim, const float* rotation,
                        const float* centroids, const float* qjl, int bits, void* out,
                        int out_dtype, void* stream);

/* ---- operator-level attention over one packed stream ---------------------------------------
 * Replaces torch.ops.turboquant.attention_scores_packed (csrc/registration.cpp:89-92,
 * csrc/cuda/attn_scores.cu:111-178, turboquant_kv/ops.py:131-194): query (bh, dim) float32,
 * one packed key stream (seq, packed_dim) shared by all bh queries; scores (bh, seq) float32,
 * UNSCALED: scores[i][s] = key_norms[s] * sum_j (R q_i)_j * centroids[code_sj]. */
int tqb_attention_scores_packed(const float* query, int64_t bh, int dim, const uint8_t* packed_keys,
                                const float* key_norms, int64_t seq, const float* centroids,
                                const float* rotation, int bits, float* scores, void* stream);

/* Replaces torch.ops.turboquant.attention_values_packed (csrc/registration.cpp:93-96,
 * csrc/cuda/attn_values.cu:121-187, turboquant_kv/ops.py:202-246):
 * out[i] = (sum_s w[i][s] * value_norms[s] * centroids[code_s,:]) @ rotation_T, out (bh, dim). */
int tqb_attention_values_packed(const float* weights, int64_t bh, int64_t seq, int dim,
                                const uint8_t* packed_values, const float* value_norms,
                                const float* centroids, const float* rotation_T, int bits,
                                float* out, void* stream);

/* ---- packed KV cache: storage layout ----------------------------------------------------------
 * The cache is NOT stored in the upstream bit-plane layout: decode attention is bound by instruction
 * issue, and turning bit planes into tensor-core operands costs more instructions than everything
 * else in the kernel.  Tokens are stored in RECORDS of 16 tokens of one (sequence, KV head), laid out
 * in the order the consuming mma.sync lanes read them (csrc/tiled_layout.cuh documents every bit):
 *     [32 lanes x dim*kbits/16 bytes of key codes][32 lanes x dim*vbits/16 bytes of value codes]
 *     [32 norms f32: 8 groups {key g, key g+8, value g, value g+8}] = 2*dim*(kbits+vbits) + 128 bytes,
 * the same codes and the same bytes per token as upstream.  A token SLOT is a flat index
 * slot = unit * pitch + position (pitch a multiple of 16); its record is slot / 16.  Contiguous cache:
 * unit = sequence * kv_heads + head, pitch = padded max_seq.  Paged cache: unit = block * kv_heads +
 * head, pitch = block_size.  tqb_kv_export / tqb_kv_import convert slots to and from upstream rows.
 *
 * vbits == 0 selects KEY-ONLY records, [32 lanes x dim*kbits/16 bytes of codes][16 norms f32] =
 * 2*dim*kbits + 64 bytes: the storage of the search index (16 database rows per record, row i in slot
 * i; 68 bytes per row at dim 128, 4 bits, as upstream).  tqb_kv_append (value = NULL), tqb_kv_export and
 * tqb_kv_import (value outputs / inputs NULL) accept them; the decode entry points do not. */
int64_t tqb_kv_record_bytes(int dim, int kbits, int vbits);

/* ---- KV-cache append ---------------------------------------------------------------------
 * Replaces the per-head quantize loop of QuantizedKVCache.append (turboquant_kv/cache.py:148-214)
 * and of _LayerQuantStore.append (turboquant_kv/hf_integration.py:111-182): quantises n key rows
 * and n value rows (each (n, dim), x_stride apart) in ONE launch, keys with (rot_k, bnd_k, kbits),
 * values with (rot_v, bnd_v, vbits), and writes input row r to token slot map(r) of `store`
 * (tqb_rowmap gives the slot; dense rows when map is NULL).  dim in {64, 128}, bits in 2..4. */
int tqb_kv_append(const void* key, const void* value, int dtype, int64_t n, int dim, int64_t x_stride,
                  const float* rot_k, const float* bnd_k, int kbits, const float* rot_v,
                  const float* bnd_v, int vbits, uint8_t* store, const tqb_rowmap* map, void* stream);

/* Upstream-layout view of n token slots: row r of the outputs is slot map(r).  k_packed (n, kbits*dim/8),
 * k_norms (n), v_packed (n, vbits*dim/8), v_norms (n); any output may be NULL.  This is what backs the
 * upstream attributes QuantizedKVCache._key_packed / _key_norms / ... (cache.py:89-106). */
int tqb_kv_export(const uint8_t* store, int64_t n, int dim, int kbits, int vbits, const tqb_rowmap* map,
                  uint8_t* k_packed, float* k_norms, uint8_t* v_packed, float* v_norms, void* stream);

/* Inverse of tqb_kv_export: writes upstream-layout rows into token slots (inputs may be NULL). */
int tqb_kv_import(uint8_t* store, int64_t n, int dim, int kbits, int vbits, const tqb_rowmap* map,
                  const uint8_t* k_packed, const float* k_norms, const uint8_t* v_packed,
                  const float* v_norms, void* stream);

/* ---- fused decode attention over a packed KV cache ------------------------------------------
 * Replaces QuantizedKVCache.attention_scores -> softmax -> attention_values
 * (turboquant_kv/cache.py:282-339, vllm_plugin/__init__.py:391-403) and the dequantise-all step
 * of TurboQuantCache.update (turboquant_kv/hf_integration.py:373-375) for one new token per
 * sequence, without materialising dense K/V.
 *
 * query (batch, q_heads, dim) of q_dtype; q_heads = group * kv_heads, query head h uses KV head
 * h / group.  out (batch, q_heads, dim) of out_dtype.  softmax(scale * q.k) over the first
 * seq_lens[b] tokens (device int32[batch]); max_len (host) >= every seq_lens[b].
 *
 * store: the record store described above.  Contiguous cache (block_tables == NULL): unit =
 * b * kv_heads + head, `max_seq` = token pitch of a unit (multiple of 16).  Paged cache: block_tables
 * (batch, max_blocks) int32 device, block_size a multiple of 16.
 *
 * dim in {64, 128}, kbits / vbits in 2..4, group <= 8.  One kernel launch per call: a grid of at most one
 * CTA per SM whose CTAs wait (bounded) for each other's partial results at the end, so it expects to be
 * resident as a whole -- do not run it beside a kernel that occupies SMs for an unbounded time.
 *
 * workspace: device scratch of at least tqb_decode_attention_workspace_bytes(...) bytes, 256-byte
 * aligned, not shared between calls that may overlap on the device.  The caller ZEROES it once before
 * its first use (cudaMemsetAsync); after that the kernel keeps its counters clean by itself.  Its first
 * 4 bytes are a status word in which the kernel only ever SETS bits (TQB_DECODE_* below); the caller
 * reads and clears it.  After TQB_DECODE_WAIT_EXPIRED or TQB_DECODE_NO_SMEM the results of that call
 * are invalid and the whole workspace must be zeroed again before the next call.
 *
 * Lengths are clamped on the device: a seq_lens[b] that is negative or exceeds max_len (a stale host
 * bound) is treated as 0 / max_len and reported with TQB_DECODE_LEN_CLAMPED; nothing is read beyond
 * max_len tokens of a unit. */
#define TQB_DECODE_WAIT_EXPIRED 1 /* a bounded device-side wait ran out: results invalid */
#define TQB_DECODE_NO_SMEM 2      /* the shared-memory plan did not fit: results invalid */
#define TQB_DECODE_UNIT_FULL 4    /* tqb_decode_step: a unit was full, its new token was not stored */
#define TQB_DECODE_LEN_CLAMPED 8  /* a sequence length outside [0, max_len] was clamped */
size_t tqb_decode_attention_workspace_bytes(int batch, int q_heads, int kv_heads, int dim,
                                            int64_t max_len);
int tqb_decode_attention(const void* query, int q_dtype, int batch, int q_heads, int kv_heads,
                         int dim, const uint8_t* store, int64_t max_seq,
                         const int32_t* seq_lens, int64_t max_len, const int32_t* block_tables,
                         int max_blocks, int block_size, const float* rot_k, const float* cent_k,
                         int kbits, const float* rot_v, const float* cent_v, int vbits, float scale,
                         void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                         void* stream);

/* One whole decode step of a layer in ONE launch: the new token's key and value of every
 * (sequence, KV head) are quantised and stored at position seq_lens[b] of their unit (what
 * QuantizedKVCache.append, turboquant_kv/cache.py:116-184, does for one token), the queries are
 * rotated, attention runs over seq_lens[b] + 1 tokens, and seq_lens[b] is advanced by one at the end
 * (device side, so a captured CUDA graph of the step can be replayed).
 * query (batch, q_heads, dim), key / value (batch, kv_heads, dim) with kv_stride elements between
 * (sequence, head) rows, all of `dtype`; contiguous caches only (unit pitch max_seq); max_len (host) >=
 * every seq_lens[b] + 1.  The stored codes equal those tqb_kv_append stores.  A unit that is already
 * full (seq_lens[b] == max_seq) stores nothing, keeps its length and sets TQB_DECODE_UNIT_FULL; a
 * position at or beyond max_len (stale host bound) is not stored either (TQB_DECODE_LEN_CLAMPED).
 * Workspace as for tqb_decode_attention (same size query, with max_len counting the new token). */
int tqb_decode_step(const void* query, const void* key, const void* value, int dtype, int64_t kv_stride,
                    int batch, int q_heads, int kv_heads, int dim, uint8_t* store, int64_t max_seq,
                    int32_t* seq_lens, int64_t max_len, const float* rot_k, const float* bnd_k,
                    const float* cent_k, int kbits, const float* rot_v, const float* bnd_v,
                    const float* cent_v, int vbits, float scale, void* workspace, size_t workspace_bytes,
                    void* out, int out_dtype, void* stream);

/* ---- packed-code inner-product scan with top-k ------------------------------------------------
 * Replaces turboquant::search_packed (csrc/core/turboquant_core.cpp:407-514) as bound by
 * turboquant_kv._core.Index.search (csrc/core/bindings.cpp:100-135) and
 * TurboQuantIndex._search_mse (turboquant_kv/search.py:206-227).
 * queries (nq, dim) float32; packed (n, packed_dim); norms (n); out_scores (nq, k) float32
 * descending, out_ids (nq, k) int64 = row + id_offset; ties ordered by ascending id; slots beyond
 * n are filled with -inf / -1.  bits in 2..4 (1 through the generic path), dim a multiple of 8,
 * k in 1..TQB_SCAN_MAX_K. */
#define TQB_SCAN_MAX_K 256
size_t tqb_scan_topk_workspace_bytes(int nq, int64_t n, int dim, int bits, int k);
int tqb_scan_topk(const float* queries, int nq, const uint8_t* packed, const float* norms,
                  int64_t n, int dim, int bits, const float* rotation, const float* centroids,
                  int k, int64_t id_offset, void* workspace, size_t workspace_bytes,
                  float* out_scores, int64_t* out_ids, void* stream);

/* The scan over an index stored as key-only records (see "storage layout" above; filled by
 * tqb_kv_append with vbits = 0 or tqb_kv_import): same results as tqb_scan_topk on the same rows --
 * scores bit-identical to upstream search_packed, ids identical except among exactly tied scores -- at a
 * third of the instructions per row, because the codes arrive in the order the MMA lanes consume them.
 * This is what TurboQuantIndex.search (turboquant_kv/search.py:206-227) runs on for dim 64 / 128 and
 * 2-4 bits.  records: ceil(n / 16) records, 16-byte aligned; rows n..16*ceil(n/16)-1 are ignored. */
size_t tqb_scan_records_workspace_bytes(int nq, int dim, int bits, int k);
/* Host-side planning figure, no device work: how many CTAs tqb_scan_records_topk gives each group of up to
 * eight queries of a call with `groups` groups over n rows on a GPU of `sms` SMs (<= 0: the current device's).
 * One group takes every SM; many groups take few, large CTAs each, in full waves, never fewer than two. */
int tqb_scan_records_ctas_per_group(int groups, int64_t n, int sms);
int tqb_scan_records_topk(const float* queries, int nq, const uint8_t* records, int64_t n, int dim, int bits,
                          const float* rotation, const float* centroids, int k, int64_t id_offset,
                          void* workspace, size_t workspace_bytes, float* out_scores, int64_t* out_ids,
                          void* stream);

/* Prod-mode search (Algorithm 2 rows): replaces TurboQuantIndex._search_prod (turboquant_kv/search.py:229-252),
 * which dequantises every row (dequantize_prod, reference.py:472-533) and multiplies by the queries.  The scan
 * computes the same inner product from the packed rows, without the dense reconstruction:
 *     <q, x~> = norm * ( <R q, c[codes]> + sqrt(pi/2)/dim * ||r|| * <S q, signs> ),   sign = 2 * bit - 1
 * mse_packed (n, (bits-1) * ceil(dim/8)), signs (n, ceil(dim/8)), res_norms (n), norms (n); S (dim, dim) the QJL
 * matrix; `bits` is the index's bit width (MSE codes use bits - 1).  Outputs as tqb_scan_topk; scores agree
 * with upstream's float32 matrix product to rounding (its summation order is the BLAS library's). */
size_t tqb_scan_topk_prod_workspace_bytes(int nq, int64_t n, int dim, int bits, int k);
int tqb_scan_topk_prod(const float* queries, int nq, const uint8_t* mse_packed, const uint8_t* signs,
                       const float* res_norms, const float* norms, int64_t n, int dim, int bits,
                       const float* rotation, const float* centroids, const float* S, int k, int64_t id_offset,
                       void* workspace, size_t workspace_bytes, float* out_scores, int64_t* out_ids, void* stream);

/* The same scan for callers that cannot allocate a workspace (no counterpart in the reference): the
 * scratch is a fixed 4 MiB array inside the library's device image, so the call reaches no allocating
 * routine.  Meant for hosts that have already handed all free device memory to pools of their own,
 * where an allocation fails or shrinks a pool, and for latency-critical loops in which a device
 * allocation would stall every stream of the process.  Calls that need more scratch than
 * tqb_scan_topk_static_capacity() bytes are rejected with TQB_ERR_WORKSPACE and a message: a call fits
 * exactly when tqb_scan_topk_workspace_bytes(nq, n, dim, bits, k) <= the capacity (the figure grows with
 * nq, k and the GPU's SM count: about two dozen queries at k = 10 on a B200); use tqb_scan_topk beyond.
 * The first call on a device resolves the array's address (cudaGetSymbolAddress, with that device
 * current): make it early, before any stream capture is begun.  All calls on a device share the array:
 * the status word at its start is cleared on `stream` by every call, the rest is rewritten before it
 * is read; calls that may overlap on the device race on it and must be serialised by the caller. */
size_t tqb_scan_topk_static_capacity(void);
int tqb_scan_topk_static(const float* queries, int nq, const uint8_t* packed, const float* norms,
                         int64_t n, int dim, int bits, const float* rotation, const float* centroids,
                         int k, int64_t id_offset, float* out_scores, int64_t* out_ids, void* stream);

/* Merge `parts` sorted candidate lists per query (the row-sharded search: one list per shard,
 * gathered over NCCL) into the global top-k with the same ordering rule.
 * scores (nq, parts, k) float32, ids (nq, parts, k) int64 -> out (nq, k). */
int tqb_topk_merge(const float* scores, const int64_t* ids, int nq, int parts, int k,
                   float* out_scores, int64_t* out_ids, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TQB200_H_ */
