/*
 * alignedkv_b200 - C ABI of the B200-native AlignedKV decode hot path.
 *
 * One entry point per operator of the reference's torch extension (extension/csrc/KV_cache_ops.cpp:69-75).
 * A binding passes raw DEVICE pointers, the reference op's own integer arguments in the reference's order,
 * and a CUDA stream handle.  Differences from the pybind surface, all forced by a C ABI:
 *   - outputs the reference allocates with torch::empty are allocated by the caller and passed in;
 *   - tensor extents the reference reads from a tensor object (v_new.size(1)) are passed as integers;
 *   - every call returns 0 or a negative AKV_ERR_* code and never throws, allocates or synchronises.
 * All byte tensors are contiguous with the reference's layouts:
 *   K planes  first_8 [B,H,n_max_blocks,D,d_block] u8, mid_4 / last_4 [B,H,n_max_blocks,D,d_block/2] u8
 *             (extension/k_cache_file.py:45-53); adjacent TOKENS share a nibble byte, even token high nibble.
 *   V planes  first_8 [B,H,max_seq_len,D] u8, mid_4 / last_4 [B,H,max_seq_len,D/2] u8
 *             (extension/v_cache_file.py:46-54); adjacent CHANNELS share a nibble byte, even channel high nibble.
 * fp16 tensors cross as bytes, little-endian, exactly as the reference's `.view(torch.uint8)` arguments.
 * Calls are asynchronous on `stream` (a cudaStream_t cast to void*; NULL = legacy default stream) and are
 * thread-safe for distinct streams.
 */
#ifndef ALIGNEDKV_B200_H
#define ALIGNEDKV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AKV_OK 0
#define AKV_ERR_NULL (-1)        /* a required pointer is NULL */
#define AKV_ERR_SHAPE (-2)       /* negative / zero / inconsistent extent, or a shape this build does not cover */
#define AKV_ERR_ALIGN (-3)       /* a pointer is not aligned as the layout requires (16 bytes for planes) */
#define AKV_ERR_OVERFLOW (-4)    /* an extent product does not fit the index type */
#define AKV_ERR_CUDA (-5)        /* the CUDA runtime reported an error at launch; see akv_last_error() */

/* Library version of this ABI (bumped on any signature change). */
int akv_abi_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* akv_last_error(void);

/*
 * Device-side health flag (no counterpart in the reference): non-zero once a bounded wait inside a kernel of this
 * library gave up - the kernel then returned early and its output is invalid.  Never expected in a healthy run.
 * Reading it copies a word from the device, i.e. synchronises; negative values are AKV_ERR_* codes.
 */
int akv_device_error_flag(void);
/*
 * Sets the flag back to zero; returns 0 or a negative AKV_ERR_* code.  The flag is per process and device image and
 * sticky: poll it where a wrong output would matter and a synchronisation is affordable (end of a request, of a
 * benchmark run, of a test), and clear it after handling the failure.  A P.V kernel whose wait ran out also writes
 * NaN into the rows it could not finish, so an unpolled failure cannot pass for a result.
 */
int akv_device_error_clear(void);

/*
 * Launch-shape knobs for benchmarking ("k_kch" 8|16, "k_stages" 3..6, "k_wpc" 0..16, "k_gqa_kch" 8|16,
 * "timing" 0|1, "pdl" 0|1: chain the kernels of a decode step with programmatic dependent launch; exact P.V:
 * "v_impl" 0 chain kernel | 1 producer-transposed kernel, "v_nf" ring depth cap, "v_nside" side-ring rows, "v_upc"
 * rings per CTA, "v_npt" low-byte tables per head, "v_gqa_form" 0 by size | 1 a ring per query head | 2 one ring per
 * KV head; order-free P.V: "v_split_impl" 0 staged through shared memory | 1 direct loads).
 * Process-wide; results never depend on them (the order-free forms agree within their tolerance, every exact form
 * bit for bit).  Returns 0, or AKV_ERR_SHAPE for an unknown key or value.  No counterpart in the reference.
 */
int akv_set_tuning(const char* key, int value);

/*
 * Replaces k_cache_save (extension/csrc/KV_cache_ops.cpp:5-16; extension/csrc/K_cache.cu:97-164).
 * Splits fp16 keys k_new [B,seqlen,H,D] into the three K planes.  Same dispatch as the reference:
 * start_pos==0 or seqlen%d_block==0 -> writes n_blocks blocks starting at block start_pos/d_block (nothing when
 * n_blocks==0); else seqlen==1 -> writes the single token at position start_pos; any other combination is a
 * silent no-op that returns AKV_OK.  The high byte is stored, nibbles are ADDED onto the existing plane bytes
 * (mod 256) as in K_cache.cu:49-56, so planes must start zeroed.
 */
int akv_k_cache_save(void* k_first_8, void* k_mid_4, void* k_last_4, const void* k_new,
                     int bsz, int n_kv_heads, int n_blocks, int n_max_blocks, int d_head, int d_block,
                     int start_pos, int seqlen, void* stream);

/*
 * Replaces k_cache_compute (KV_cache_ops.cpp:18-32; K_cache.cu:314-395).
 * s_out: caller-allocated fp16 bytes [B,H,1,(n_blocks+1)*d_block]; only [..., :n_blocks*d_block] is written,
 * bit-identical to the reference kernel (fp16 fused multiply-add in channel order, then * half(sqrt_dim)).
 * kq [B,1,H,D] u8, kqmax [B,1,H,1] u8, q fp16 bytes [B,1,H,D].  `seqlen` is accepted and unused, as in the
 * reference.  Unlike the reference (which computes only heads below 4*floor(H/4)) every head is computed.
 * reference!=0 reads every plane.
 */
int akv_k_cache_compute(const void* k_first_8, const void* k_mid_4, const void* k_last_4,
                        const void* kq, const void* kqmax, const void* q, void* s_out,
                        int bsz, int n_kv_heads, int n_blocks, int n_max_blocks, int d_head, int d_block,
                        int seqlen, float sqrt_dim, int reference, void* stream);

/*
 * Replaces v_cache_save (KV_cache_ops.cpp:34-43; extension/csrc/V_cache.cu:44-80).
 * v_new: fp16 bytes [B,v_new_tokens,H,D]; v_new_tokens is the tensor's own token extent, which the reference
 * reads as v_new.size(1) (V_cache.cu:65).  Writes tokens [start_pos, start_pos+seq_len) with plain stores.
 */
int akv_v_cache_save(void* v_first_8, void* v_mid_4, void* v_last_4, const void* v_new,
                     int bsz, int n_local_kv_heads, int max_seq_len, int head_dim, int start_pos, int seq_len,
                     int v_new_tokens, void* stream);

/*
 * Replaces v_cache_test_compute (KV_cache_ops.cpp:45-54; V_cache.cu:125-168).
 * test_s_value fp16 bytes [B,H,1,top_max_k], test_s_index int32 bytes [B,H,1,top_max_k],
 * test_o: caller-allocated fp16 bytes [B,H,1,D].  Row index idx*top_max_k+j is clamped into
 * [0, max_seq_len-1] (the reference reads out of bounds there).
 */
int akv_v_cache_test_compute(const void* v_first_8, const void* v_mid_4, const void* v_last_4,
                             const void* test_s_value, const void* test_s_index, void* test_o,
                             int bsz, int n_local_kv_heads, int max_seq_len, int head_dim, int top_max_k,
                             void* stream);

/*
 * Replaces v_cache_compute (KV_cache_ops.cpp:56-67; V_cache.cu:310-374).
 * s: fp16 bytes, row (b,h) starts at half index (b*H+h)*s_last_dim; amin: u8 read flat at b*H+h;
 * o_out: caller-allocated fp16 bytes [B,H,1,D], bit-identical to the reference kernel (fp16 fused
 * multiply-add in token order).  reference!=0 reads every plane.
 */
int akv_v_cache_compute(const void* v_first_8, const void* v_mid_4, const void* v_last_4,
                        const void* s, const void* amin, void* o_out,
                        int bsz, int n_local_kv_heads, int max_seq_len, int head_dim, int s_last_dim,
                        int start_pos_add_seqlen, int reference, void* stream);

/*
 * One decode step of one layer in a single call: what the reference does between receiving (q, k_new, v_new) of a
 * decode token and returning the attention output - K_Cache_Class.save + decoding_compute
 * (extension/k_cache_file.py:97-118,132-159), the fp32 softmax (model/KVCache_AlignedKV.py:119-121; without a mask -
 * akv_decode_step_masked takes one) and
 * V_Cache_Class.save + decoding_compute (extension/v_cache_file.py:97-116,119-190) - with the wrapper's small
 * tensor operations folded into kernels.  All pointers are device pointers:
 *   planes as above; k_exp_max / v_exp_max [B,1,H,D] u8 (updated in place); restk / restv [B,64,H,D] fp16 residual
 *   buffers (the new token is written at row rest_len); q, k_new, v_new [B,1,H,D] fp16; out [B,1,H,D] fp16;
 *   scratch: workspace of at least akv_decode_scratch_bytes() bytes, 16-byte aligned, owned by the caller.
 * rest_len / rest_start are the residual fill count and first buffered position BEFORE this token
 * (the reference's restklen / reststartpos).  After the call the caller advances them: rest_len + 1, or
 * (0, rest_start + 64) when rest_len was 63 (this call then also wrote that block to the planes).
 * head_dim must be a multiple of 64.  Plane bytes and read decisions equal the operator-by-operator path; the
 * softmax and the residual-token dot products are fp32 like torch's but may differ from it in the last bit.
 */
int akv_decode_step(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                    void* k_exp_max, void* v_exp_max, void* restk, void* restv,
                    const void* q, const void* k_new, const void* v_new, void* out,
                    void* scratch, long long scratch_bytes,
                    int bsz, int n_heads, int head_dim, int max_seq_len, int rest_len, int rest_start,
                    int reference, void* stream);

/* Bytes of workspace akv_decode_step needs for these extents (-1 on bad extents). */
long long akv_decode_scratch_bytes(int bsz, int n_heads, int head_dim, int max_seq_len);

/*
 * Grouped-query forms (no counterpart in the reference, which asserts multi-head attention:
 * model/KVCache_AlignedKV.py:32, extension/k_cache_file.py:133, extension/v_cache_file.py:146).  `group` query heads
 * share each of the n_kv_heads KV heads; query head index = KV head * group + g.  Planes, exponent maxima and
 * residual buffers are per KV head; kq, kqmax, q, score rows, amin and outputs are per query head.  Results equal the
 * multi-head operators run on a cache whose KV heads were repeated `group` times, while every plane byte is
 * fetched from HBM once per group.
 * flags: AKV_STEP_REFERENCE reads every plane; AKV_STEP_ORDER_FREE selects the P.V kernel that splits the token axis
 * across CTAs and accumulates in fp32 (same read decisions and substitute constants, different summation order:
 * not bit-identical to the reference's fp16 token-order chain, closer to exact arithmetic; head_dim 128 only; needs a
 * workspace of akv_v_cache_compute_scratch_bytes() bytes); AKV_STEP_NO_APPEND (decode step only) leaves the cache
 * untouched - the new token belongs to another shard of the sequence.
 */
#define AKV_STEP_REFERENCE 1
#define AKV_STEP_ORDER_FREE 2
#define AKV_STEP_NO_APPEND 4
#define AKV_STEP_TRACK_MAXIMA 8   /* with AKV_STEP_NO_APPEND (akv_shard_step): the new token still updates the exponent maxima */
int akv_k_cache_compute_gqa(const void* k_first_8, const void* k_mid_4, const void* k_last_4,
                            const void* kq, const void* kqmax, const void* q, void* s_out,
                            int bsz, int n_kv_heads, int group, int n_blocks, int n_max_blocks, int d_head, int d_block,
                            int seqlen, float sqrt_dim, int reference, void* stream);
int akv_v_cache_compute_gqa(const void* v_first_8, const void* v_mid_4, const void* v_last_4,
                            const void* s, const void* amin, void* o_out, void* scratch, long long scratch_bytes,
                            int bsz, int n_kv_heads, int group, int max_seq_len, int head_dim, int s_last_dim,
                            int start_pos_add_seqlen, int flags, void* stream);
long long akv_v_cache_compute_scratch_bytes(int bsz, int n_kv_heads, int group, int n_tokens);

/*
 * akv_decode_step with grouped-query attention, the choice of P.V kernel, and an optional packed result for
 * sequence-sharded caches.  q and out are [B,1,n_kv_heads*group,D]; k_new, v_new, the residual buffers and exponent
 * maxima are per KV head.  packed_out (may be NULL): fp32 [B*Hq, D+2] rows (maximum score, sum of exponentials,
 * output[0..D-1]) over THIS cache's tokens - what akv_lse_merge combines across shards; `out` may be NULL when only
 * the packed result is wanted.  With AKV_STEP_NO_APPEND k_new / v_new may be NULL and rest_len / rest_start stay
 * as they are.
 */
int akv_decode_step_ex(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                       void* k_exp_max, void* v_exp_max, void* restk, void* restv,
                       const void* q, const void* k_new, const void* v_new, void* out, void* packed_out,
                       void* scratch, long long scratch_bytes,
                       int bsz, int n_kv_heads, int group, int head_dim, int max_seq_len, int rest_len, int rest_start,
                       int flags, void* stream);
long long akv_decode_scratch_bytes_ex(int bsz, int n_kv_heads, int group, int head_dim, int max_seq_len, int flags);

/*
 * akv_decode_step_ex with the attention mask the reference adds to the scores before the softmax
 * (model/KVCache_AlignedKV.py:119-120: `scores[..., :start_pos+seqlen] += mask`).  mask (NULL = none): additive fp16
 * values, one row per batch row, row b at mask + b * mask_stride halves (mask_stride 0 = one row for the whole batch),
 * broadcast over the heads; entry t applies to cached position t, entries [0, cache length after this step) are read.
 * The addition happens in fp16 (one rounding) like the reference's in-place add on fp16 tensors, and the softmax then runs
 * in fp32 over the masked scores - a left-padded batch passes its usual mask row with the most negative fp16 value at the
 * padding positions, whose probabilities then come out as zero.
 */
int akv_decode_step_masked(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                           void* k_exp_max, void* v_exp_max, void* restk, void* restv,
                           const void* q, const void* k_new, const void* v_new, void* out, void* packed_out,
                           const void* mask, long long mask_stride, void* scratch, long long scratch_bytes,
                           int bsz, int n_kv_heads, int group, int head_dim, int max_seq_len, int rest_len, int rest_start,
                           int flags, void* stream);

/*
 * Prompt ingestion in one pass: K_Cache_Class.save + V_Cache_Class.save for start_pos == 0
 * (extension/k_cache_file.py:76-96, extension/v_cache_file.py:79-96; writers extension/csrc/K_cache.cu:19-58,
 * extension/csrc/V_cache.cu:17-41).  k, v: fp16 [B,seqlen,H,D].  Writes the whole 64-token blocks to the planes (K
 * nibbles are added, so planes must start zeroed), the remaining seqlen % 64 tokens to rows 0.. of the residual
 * buffers [B,64,H,D] (other rows are left as they are), and the exponent field of the SIGNED per-channel maximum
 * over the prompt to k_exp_max / v_exp_max [B,1,H,D] (the reference takes the signed maximum here and magnitudes on
 * decode).  Afterwards rest_len = seqlen % 64, rest_start = seqlen - rest_len.  head_dim: multiple of 32, <= 256.
 * scratch: akv_prefill_scratch_bytes() bytes, 16-byte aligned.
 */
int akv_prefill(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* k, const void* v,
                void* scratch, long long scratch_bytes, int bsz, int n_kv_heads, int head_dim, int max_seq_len,
                int seqlen, void* stream);
long long akv_prefill_scratch_bytes(int bsz, int n_kv_heads, int head_dim, int seqlen);

/*
 * Roll the cache back to an earlier length (no counterpart in the reference; used to drop speculative tokens and to
 * replay a step).  The caller keeps copies of the exponent maxima taken at the earlier length and its own
 * (rest_len, rest_start); this call puts the maxima back and clears the K nibble planes of the blocks
 * [first_block, first_block + n_blocks) that were written since - the K writer adds nibbles, so a block must be zero
 * before it is written again.  Nothing else needs undoing: high bytes, V planes and residual rows are overwritten by
 * plain stores when the positions are appended again.
 */
int akv_rollback(void* k_mid_4, void* k_last_4, void* k_exp_max, void* v_exp_max, const void* k_exp_saved,
                 const void* v_exp_saved, int bsz, int n_kv_heads, int head_dim, int max_seq_len, int first_block,
                 int n_blocks, void* stream);

/*
 * Log-sum-exp merge of the packed results of n_ranks shards of one sequence (no counterpart in the reference, which
 * is single-device).  packed: fp32 [n_ranks, rows, head_dim+2] as gathered from the shards (rows = B*Hq);
 * out: fp16 [rows, head_dim] = sum_g w_g o_g with w_g = l_g exp(m_g - M) / sum_g' l_g' exp(m_g' - M), M = max_g m_g.
 * Shards with l = 0 (no tokens) are ignored.
 */
int akv_lse_merge(const void* packed, void* out, int n_ranks, int rows, int head_dim, void* stream);

/*
 * The same merge with the exchange inside the kernel, through peer memory (no counterpart in the reference): one launch
 * per decode step on every rank replaces the all-gather of the shards' packed results and akv_lse_merge.
 * Every rank (one process per GPU of one node, at most 8) owns an exchange buffer of akv_exchange_bytes() bytes,
 * zero at the start, and maps the other ranks' buffers:
 *   akv_peer_alloc   device memory of the current device (cleared) and the 64-byte handle another process opens it by;
 *   akv_peer_open    another process's buffer, by the handle that process got (CUDA IPC; the address is valid in the
 *                    calling process only; peer access between the two GPUs is enabled on first use);
 *   akv_peer_close / akv_peer_free   undo the two (close every mapping of a buffer before its owner frees it).
 * Limits: head_dim at most 256, and at most two rows per SM (every row's CTA has to be resident at once).
 * Buffer layout for R ranks, rows = B*Hq, W = head_dim + 2 (head_dim at most 256): 8-byte words [2][R][rows][W], a word
 * = (the bits of one float of a record, the epoch it belongs to); slot g is written by rank g; two epochs deep (index
 * epoch & 1).  A float and its flag travel in one aligned 8-byte store, which is atomic, so neither side needs a fence.
 * akv_exchange_merge(bufs, rank, ...): bufs[g] = the calling process's address of rank g's buffer (bufs[rank] its
 * own).  record: this rank's fp32 [rows, head_dim+2] as akv_decode_step_ex packs it; out: fp16 [rows, head_dim] as
 * akv_lse_merge.  epoch: 1 for the first step, one more each step, the same on every rank.  The kernel stores the
 * record's words into slot `rank` of every buffer, reads the words of all ranks from its own buffer until each carries
 * the epoch, and merges.  The wait is bounded by timeout_ms (1..10000): when it runs out, the kernel raises the device
 * error flag (bit 2, akv_device_error_flag), writes zeros to `out` and returns; the context stays usable.  Ranks must
 * be launched on different GPUs: a rank's kernel waits for the others.
 */
#define AKV_PEER_HANDLE_BYTES 64
long long akv_exchange_bytes(int n_ranks, int rows, int head_dim);
int akv_peer_alloc(long long bytes, void** ptr, void* handle);
int akv_peer_open(const void* handle, void** ptr);
int akv_peer_close(void* ptr);
int akv_peer_free(void* ptr);
int akv_exchange_merge(void* const* bufs, int rank, int n_ranks, const void* record, void* out, int rows,
                       int head_dim, unsigned int epoch, int timeout_ms, void* stream);

/*
 * akv_decode_step_ex over one shard of a sequence-sharded cache with that exchange inside the step's last kernel (no
 * counterpart in the reference): the kernel that finishes a (batch, query head) row's packed record also stores it
 * into every rank's exchange buffer, waits for the other ranks' records of the row and writes the merged row - no
 * launch and no collective between the shard's result and the attention output.  Arguments as akv_decode_step_ex
 * (packed_out: this shard's records, required; flags: AKV_STEP_ORDER_FREE / AKV_STEP_NO_APPEND as there), then the
 * exchange as akv_exchange_merge; merged_out: fp16 [bsz, 1, n_kv_heads*group, head_dim], the same on every rank.
 */
int akv_decode_step_exchange(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4,
                             void* v_last_4, void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q,
                             const void* k_new, const void* v_new, void* merged_out, void* packed_out, void* scratch,
                             long long scratch_bytes, int bsz, int n_kv_heads, int group, int head_dim, int max_seq_len,
                             int rest_len, int rest_start, int flags, void* const* bufs, int rank, int n_ranks,
                             unsigned int epoch, int timeout_ms, void* stream);

/*
 * akv_decode_step for callers that cannot allocate device memory (no counterpart in the reference).
 * Same arguments and results as akv_decode_step, minus the workspace: it lives in a fixed array of
 * AKV_NOALLOC_SCRATCH_BYTES bytes of device global memory inside the library image, which every GPU that loads the
 * library keeps reserved until the process exits.  The call itself performs no cudaMalloc / cudaFree and calls no
 * allocating library routine.  Meant for hosts whose device memory was handed out once at start-up and is locked
 * afterwards, and for code that runs where an allocation (which synchronises the device) is not allowed.
 *  - Extents whose workspace (akv_decode_scratch_bytes) exceeds AKV_NOALLOC_SCRATCH_BYTES are rejected with
 *    AKV_ERR_SHAPE.  The benchmark's "timing" knob (which creates CUDA events) is ignored by this entry point.
 *  - With CUDA's lazy module loading the FIRST launch of each kernel of the step may allocate inside the driver; the
 *    block writers first run on the step that completes a 64-token block.  A caller that must not allocate later warms
 *    up with steps that cross a block boundary (the residual count passing 63) before its memory is locked.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *    current); make that first call before any stream capture begins.
 *  - All calls on a device share the one array and find the previous call's bytes in it.  Nothing in it has to
 *    start at zero (every region is fully written before it is read within a call), but two calls that overlap on
 *    the GPU - different streams, or different caches on one stream without ordering - race on it: serialise them.
 */
#define AKV_NOALLOC_SCRATCH_BYTES (8u << 20)
int akv_decode_step_noalloc(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4,
                            void* v_last_4, void* k_exp_max, void* v_exp_max, void* restk, void* restv,
                            const void* q, const void* k_new, const void* v_new, void* out,
                            int bsz, int n_heads, int head_dim, int max_seq_len, int rest_len, int rest_start,
                            int reference, void* stream);

/*
 * One decode step over a shard of a sequence-sharded cache, cut into four phases with an exchange between them so that
 * every shard takes the read decisions one device holding the whole sequence would take (no counterpart in the
 * reference, which is single-device).  rows = bsz * n_kv_heads * group; a chunk is 4096 scores; local chunks =
 * ceil(((quantized local tokens after the step) / 64 + 1) * 64 / 4096).
 *   phase 1: append (last shard) or, with AKV_STEP_NO_APPEND | AKV_STEP_TRACK_MAXIMA, only take the new token into the
 *            exponent maxima; q.K^T; chunk statistics            -> exch_out float [rows][local chunks][2]
 *   phase 2: exch_in float [rows][chunks_total][2] (every shard's statistics, sequence order); probabilities of the
 *            local tokens and residue-class candidates           -> exch_out u32 [rows][local chunks][32] values, then
 *                                                                   i32 [rows][local chunks][32] positions / 32
 *   phase 3: exch_in the same two arrays over chunks_total; winners; high-byte rows of the winners held here
 *                                                                -> exch_out bytes [rows][32][head_dim]
 *   phase 4: exch_in the shards' row buffers added up; probe, threshold bytes, order-free P.V, residual tokens
 *                                                                -> exch_out float [rows][head_dim + 2]; words 2.. are
 *                                                                   this shard's part of the output (parts add up)
 * Layout: a phase 1 / 2 output has a row stride of out_chunks chunks (0 = the local count; a caller that pads every
 * rank to a common count pre-fills the padding with empty chunks: statistics (-inf, 0), candidates 0).  A phase 2 / 3
 * input is n_ranks such buffers one after the other, as an all-gather leaves them (chunks_total = n_ranks x the common
 * count), or with n_ranks == 1 one buffer over all chunks in sequence order.
 * token_base: position of local token 0 in the whole sequence (a multiple of 4096).  All phases take the state before
 * the step; the caller advances rest_len / rest_start after phase 4 as for akv_decode_step_ex.  scratch: at least
 * akv_decode_scratch_bytes_ex(..., AKV_STEP_ORDER_FREE) bytes, untouched between the phases.  head_dim 128.
 */
int akv_shard_step(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                   void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q, const void* k_new,
                   const void* v_new, const void* exch_in, void* exch_out, void* scratch, long long scratch_bytes,
                   int bsz, int n_kv_heads, int group, int head_dim, int max_seq_len, int rest_len, int rest_start,
                   int token_base, int chunks_total, int n_ranks, int out_chunks, int flags, int phase, void* stream);

/*
 * Benchmark instrumentation (no counterpart in the reference): with akv_set_tuning("timing", 1), akv_decode_step
 * records CUDA events around its q.K^T and P.V launches.  akv_timing_read returns how many steps were recorded
 * since akv_timing_reset and their median launch durations in microseconds; synchronise the stream first.
 */
int akv_timing_reset(void);
int akv_timing_read(double* k_us, double* v_us);

/*
 * Number of kernels this library has launched in this process so far (no counterpart in the reference); a caller
 * takes the difference around a region to know how many of the library's kernels ran in it.
 */
long long akv_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* ALIGNEDKV_B200_H */
