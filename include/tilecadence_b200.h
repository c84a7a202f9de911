/* C ABI of the B200 (sm_100a) attention operators.
 *
 * Each entry point replaces one dispatcher op that TileCadence's generated extensions register
 * with TORCH_LIBRARY, with the tensors flattened to raw device pointers, explicit sizes and
 * element strides. Conventions shared by every call:
 *   - returns TC_OK (0) or a TC_ERR_* code; tc_last_error() gives the thread-local message
 *     (the counterpart of the reference's TORCH_CHECK text);
 *   - `device` is the CUDA ordinal that owns every pointer, `stream` a cudaStream_t (NULL = legacy
 *     default stream). Work is enqueued on that stream; there is no host synchronisation and no
 *     host read of device lengths (tilecadence/cuda/decode/decode.cu:50-52);
 *   - the caller owns and preallocates every buffer, workspaces included; nothing is allocated per
 *     call. The library keeps one small per-device block (split tickets and a kernel status word)
 *     that it allocates on the first call for a device, so the first call on a device must happen
 *     outside CUDA-graph capture;
 *   - layouts are the reference's: Q/O [B,T,Hq,128], K/V and caches [B,*,Hkv,128], 16-bit
 *     elements, last dimension contiguous; LSE fp32, natural log; four query heads per KV head;
 *   - only compute capability 10.x devices are accepted: there is no fallback path.
 */
#ifndef TILECADENCE_B200_H
#define TILECADENCE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TC_OK 0
#define TC_ERR_INVALID 1 /* argument check failed (shape, stride, alignment, aliasing, range) */
#define TC_ERR_CUDA 2    /* a CUDA runtime/driver call failed */
#define TC_ERR_DEVICE 3  /* not an sm_100 device */
#define TC_ERR_KERNEL 4  /* a kernel reported a bounded wait that expired */

#define TC_ABI_VERSION 1

/* Thread-local text of the last failure on this host thread ("" if none). */
const char* tc_last_error(void);
int tc_abi_version(void);

/* Reads and clears the kernel status of a device (synchronises the device). *status is 0 when no
 * kernel wait expired since the previous call, else the first code found. It covers the library's
 * per-device block (if a decode call created it) and the status word of tc_decode_forward_out_static;
 * it never allocates: a device on which no call has been made yet reports 0. Has no counterpart in
 * the reference, whose kernels have no bounded waits. */
int tc_device_status(int device, int32_t* status);

/* ---------------------------------------------------------------------------------- prefill
 * Causal GQA prefill, BF16, O + LSE.
 *
 * workspace_spec replaces `workspace_spec(q,k,v,num_splits,mapping,causal) -> int[3]`
 * (tilecadence/cuda/prefill/binding.cpp:12, prefill.cu:106-120): spec = {1, 0, 0}.
 * num_splits must be 0, mapping 0 or 1, causal non-zero, batch 1 or 4, 128 <= tokens <= 32768
 * (prefill.cu:69-74,109-114). q_heads is 32 in the reference; a multiple of 4 up to 32 is accepted
 * so that a rank can hold a KV-head-group shard.
 */
int tc_prefill_workspace_spec(int device, int64_t batch, int64_t tokens, int64_t q_heads, int64_t num_splits,
                              int64_t mapping, int causal, int64_t spec[3]);

/* Replaces `forward_out(q,k,v,out!,lse!,workspace_o!,workspace_lse!,num_splits,mapping,scale,causal)`
 * (tilecadence/cuda/prefill/binding.cpp:11, prefill.cu:122-152, common.cuh:36-78).
 * q [B,T,Hq,128], k/v [B,T,Hq/4,128] with element strides {batch,row,head} (multiples of 8, last
 * dimension contiguous, 16-byte aligned bases); out contiguous like q; lse contiguous [B,Hq,T].
 * workspace_*_elems must be 0 (single split). mapping 1 stages the per-row LSE of both heads in the
 * released terminal K stage at the planner's offsets; mapping 0 uses a dedicated staging area. Both
 * give bit-identical results.
 */
int tc_prefill_forward_out(int device, void* stream, const void* q, const int64_t q_strides[3], const void* k,
                           const int64_t k_strides[3], const void* v, const int64_t v_strides[3], void* out,
                           float* lse, int64_t workspace_o_elems, int64_t workspace_lse_elems, int64_t batch,
                           int64_t tokens, int64_t q_heads, int64_t num_splits, int64_t mapping, double scale,
                           int causal);

/* Prefill for launches that cannot fill the GPU with one CTA per query tile (a KV-head-group shard of a
 * sequence, few heads): every 128-row query tile is given to two CTAs that each take half of its key tiles,
 * and the CTA that finishes a head second merges the other's normalised O and LSE into its own (the
 * LSE-weighted merge of the decode split) before it stores. Same tensors and checks as tc_prefill_forward_out
 * (causal, num_splits 0). `workspace` is caller-owned, 256-byte aligned, of at least
 * tc_prefill_key_split_workspace_bytes(batch, tokens, q_heads) bytes and disjoint from the tensors; its ticket
 * words are cleared on the stream by this call. key_splits: 1 = one CTA per tile (the workspace is unused and
 * the result is bit-identical to tc_prefill_forward_out), 2 = two, 0 = chosen from the tile and SM counts;
 * *key_splits_used (may be NULL) receives the choice. With two CTAs the accumulation order differs, so results
 * agree with the single-CTA result to rounding, not bit for bit. No counterpart in the reference, whose
 * prefill requires a single split (prefill.cu:109). */
int tc_prefill_key_split_workspace_bytes(int64_t batch, int64_t tokens, int64_t q_heads, int64_t* bytes);
int tc_prefill_key_split_forward_out(int device, void* stream, const void* q, const int64_t q_strides[3], const void* k,
                                     const int64_t k_strides[3], const void* v, const int64_t v_strides[3], void* out,
                                     float* lse, void* workspace, int64_t workspace_bytes, int64_t batch,
                                     int64_t tokens, int64_t q_heads, int64_t mapping, double scale, int64_t key_splits,
                                     int64_t* key_splits_used);

/* Replaces `resources(q,k,v,num_splits,mapping,causal) -> int[]` (prefill.cu:154-167): 12 header
 * values, 8 kernel attributes (threads, dynamic smem, static smem, registers/thread, local
 * bytes/thread, binary version, PTX version, active CTAs/SM), 8 zeros, 18 layout values. */
int tc_prefill_resources(int device, const int64_t q_strides[3], const int64_t k_strides[3],
                         const int64_t v_strides[3], int64_t batch, int64_t tokens, int64_t q_heads,
                         int64_t num_splits, int64_t mapping, int causal, int64_t* values, int64_t capacity,
                         int64_t* count);

/* ---------------------------------------------------------------------------------- decode
 * Split-KV decode for one new token per sequence with the KV-cache append fused in.
 *
 * Replaces `workspace_spec(q,kcache,old_lengths,num_splits,mapping,append) -> int[3]`
 * (tilecadence/cuda/decode/binding.cpp:21, decode.cu:76-83): spec = {splits,
 * splits*B*Hq*128, splits*B*Hq} fp32 elements (zeros when splits == 1). num_splits 0 picks the
 * split count from the SM count; a positive value (<= 128) is used as given.
 */
int tc_decode_workspace_spec(int device, int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits,
                             int64_t mapping, int append, int64_t spec[3]);

/* Replaces `forward_out(q,kcache!,vcache!,knew,vnew,old_lengths,out!,lse!,workspace_o!,
 * workspace_lse!,num_splits,mapping,append)` (tilecadence/cuda/decode/binding.cpp:17-20,
 * decode.cu:158-193). q/out [B,1,Hq,128] BF16 contiguous, caches [B,capacity,Hkv,128] contiguous,
 * knew/vnew [B,1,Hkv,128], old_lengths int32[B] on the device with 0 <= old_lengths[b] <= capacity-1
 * when append is set; lse fp32 [B,Hq,1]. With append, row old_lengths[b] of both caches receives the
 * new K/V row (bit copy) and keys [0, old_lengths[b]] are attended; without, keys [0, old_lengths[b]).
 * Softmax scale is 128^-0.5 (decode.cu:106). The split partials are merged inside the same launch
 * by the last CTA to finish each (batch, KV head). All ten buffers must be pairwise disjoint
 * (decode.cu:176-177). Calls that share a device must not overlap on the GPU (they share tickets).
 */
int tc_decode_forward_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                          const void* vnew, const int32_t* old_lengths, void* out, float* lse,
                          float* workspace_o, int64_t workspace_o_elems, float* workspace_lse,
                          int64_t workspace_lse_elems, int64_t batch, int64_t capacity, int64_t kv_heads,
                          int64_t num_splits, int64_t mapping, int append);

/* tc_decode_forward_out with option flags. TC_DECODE_CACHE_STABLE is the caller's promise that the kernel
 * launched immediately before this call on the same stream writes none of: the cache rows below
 * old_lengths[b], old_lengths itself (and, where used, index tables). The launch uses programmatic dependent
 * launch; with the flag the length read and the K/V stream start while that preceding kernel is still
 * finishing (the first tiles into the shared-memory ring, the others as prefetches into L2), and only q, knew,
 * vnew and all writes wait for it. Typical cases: the preceding kernel is the projection that produces q / knew
 * / vnew, or the decode step of another layer (other caches). TC_DECODE_PREFIX_STABLE is the narrower promise
 * for a preceding kernel that was the previous decode step of the SAME caches: it may have written row
 * old_lengths[b] - 1 and nothing else of the above; then only the tiles that end below that row are fetched
 * early. The two flags are alternatives. A CTA whose share of the cache is longer than 32 tiles (2048 rows) makes
 * no use of either promise: such a launch is bandwidth-bound from end to end and an early start only competes with
 * the preceding kernel. If the promise does not hold, results are undefined; flags = 0 is tc_decode_forward_out.
 * No counterpart in the reference. */
#define TC_DECODE_CACHE_STABLE 1
#define TC_DECODE_PREFIX_STABLE 2
int tc_decode_forward_out_flags(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                                const void* vnew, const int32_t* old_lengths, void* out, float* lse,
                                float* workspace_o, int64_t workspace_o_elems, float* workspace_lse,
                                int64_t workspace_lse_elems, int64_t batch, int64_t capacity, int64_t kv_heads,
                                int64_t num_splits, int64_t mapping, int append, int64_t flags);

/* Allocation-free decode step. It has no counterpart in the reference; it exists for callers that
 * are not allowed to allocate device memory at all: code running inside a fixed memory budget that
 * was carved up at start-up (an inference server whose allocator owns every byte), code that must not
 * disturb a caching allocator's state, or a call site where cudaMalloc's implicit synchronisation is
 * unacceptable. Arguments and results are those of tc_decode_forward_out without the workspace: the
 * split partials, the split tickets and the status word live in a 2.1 MiB array that is part of the
 * library image (every GPU that loads the library holds it until the process exits). Limits: batch *
 * query heads <= 128 rows and at most 32 splits; anything larger is rejected with TC_ERR_INVALID (use
 * tc_decode_forward_out with your own workspace). num_splits 0 picks the usual split count, capped at 32.
 * The call makes no cudaMalloc/cudaFree and uses no allocating library routine; it encodes its tensor
 * maps on the stack and clears the tickets with cudaMemsetAsync on `stream`. The first call on a
 * device looks up the array's device address (cudaGetSymbolAddress, once per device): make that first
 * call before any stream capture. All calls on a device share the one array, which keeps the previous
 * call's partials: two calls that overlap on the GPU (different streams) race; serialise them.
 * A bounded wait that expires inside a static call is recorded in a status word of the same array (not in
 * the per-device block, which such a caller never creates). The word keeps the first code until it is read:
 * tc_device_status reads and clears it without allocating, and tc_decode_static_status_word gives its device
 * address (also without allocating; it does the same first-call address look-up) to callers that prefer to
 * copy the 4 bytes on a stream of their own. */
int tc_decode_forward_out_static(int device, void* stream, const void* q, void* kcache, void* vcache,
                                 const void* knew, const void* vnew, const int32_t* old_lengths, void* out,
                                 float* lse, int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits,
                                 int64_t mapping, int append);
int tc_decode_static_status_word(int device, int32_t** word);

/* KV-sequence-sharded variant for multi-GPU decode; no counterpart in the reference (it has no
 * distributed path). The caches hold global rows [kv_shard_start, kv_shard_start + capacity) of each
 * sequence; old_lengths stay global. The shard that owns row old_lengths[b] performs the append.
 * Outputs are this shard's normalised partial O (fp32 [B,Hq,128]) and partial LSE (fp32 [B,Hq],
 * -inf where the shard holds no visible key), ready for an all-gather + tc_combine_partials. */
int tc_decode_partial_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                          const void* vnew, const int32_t* old_lengths, float* partial_o, float* partial_lse,
                          float* workspace_o, int64_t workspace_o_elems, float* workspace_lse,
                          int64_t workspace_lse_elems, int64_t batch, int64_t capacity, int64_t kv_heads,
                          int64_t num_splits, int64_t mapping, int append, int64_t kv_shard_start);

/* LSE-weighted merge of `parts` partial results: the arithmetic of the split combine the reference
 * launches after its decode kernel (decode.cu:131-140): LSE = ln sum_s exp(LSE_s),
 * O = sum_s exp(LSE_s - LSE) O_s. Part s has its O at partial_o + s*part_stride_o (fp32
 * [rows,128]) and its LSE at partial_lse + s*part_stride_lse (fp32 [rows]); strides are in
 * elements, so the parts may sit inside one gathered buffer. out BF16 [rows,128], lse fp32 [rows].
 * Rows with no contribution give O = 0, LSE = +inf. */
int tc_combine_partials(int device, void* stream, const float* partial_o, const float* partial_lse, int64_t parts,
                        int64_t rows, int64_t part_stride_o, int64_t part_stride_lse, void* out, float* lse);

/* Decode step over indexed caches: the two indirections the reference's split kernel carries
 * (ab_fused_splitkv.cuh:92-103: `cache_batch_idx`, and `block_table` + `page_block_size`) but its host
 * code never sets. Everything not listed is as in tc_decode_forward_out.
 *   block_table != NULL   paged caches: kcache/vcache are BF16 [cache_slots, slot_rows, Hkv, 128] (pages of
 *                         slot_rows rows, a multiple of 64); row r of sequence b lives in page
 *                         block_table[b*block_table_stride + r/slot_rows] at row r % slot_rows. The
 *                         sequence capacity is pages_per_seq * slot_rows; old_lengths[b] must be below it.
 *                         cache_batch_idx must be NULL.
 *   block_table == NULL   cache_batch_idx (int32 [B], required) picks the cache slot of sequence b;
 *                         caches are [cache_slots, slot_rows = capacity, Hkv, 128]; pages_per_seq is ignored.
 * Table entries are read on the device; values outside [0, cache_slots) are clamped so that no access
 * leaves the cache allocation. The appended row is written to its page. Two sequences must not map to
 * the same page or slot. Size the split workspace with tc_decode_workspace_spec(batch, capacity, ...). */
int tc_decode_indexed_forward_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                                  const void* vnew, const int32_t* old_lengths, void* out, float* lse,
                                  float* workspace_o, int64_t workspace_o_elems, float* workspace_lse,
                                  int64_t workspace_lse_elems, int64_t batch, int64_t cache_slots, int64_t slot_rows,
                                  int64_t kv_heads, int64_t num_splits, int64_t mapping, int append,
                                  const int32_t* block_table, int64_t block_table_stride, int64_t pages_per_seq,
                                  const int32_t* cache_batch_idx);

/* tc_decode_forward_out for callers whose q and knew are NOT yet rotated: the step before attention in the
 * reference's pipeline ("the host passes pre-rotated Q/K", ab_fused_splitkv.cuh:189) folded into the decode
 * launch. The kernel applies rotate-half rotary position embedding to every query head and to the new K
 * row for position old_lengths[b], attends with the rotated q, and appends the rotated K row (V is copied
 * as is). rope_cos / rope_sin are FP32 [rope_positions, 64] (the 64 distinct frequencies; row = position,
 * clamped to the table), 16-byte aligned. For i < 64: x'[i] = x[i]*cos[i] - x[i+64]*sin[i],
 * x'[i+64] = x[i+64]*cos[i] + x[i]*sin[i], every product and sum rounded to FP32 separately and the result
 * rounded to BF16 (round to nearest even), so a host restatement reproduces the appended row bit for bit. */
int tc_decode_rope_forward_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                               const void* vnew, const int32_t* old_lengths, void* out, float* lse, float* workspace_o,
                               int64_t workspace_o_elems, float* workspace_lse, int64_t workspace_lse_elems,
                               int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits, int64_t mapping,
                               int append, const float* rope_cos, const float* rope_sin, int64_t rope_positions);

/* Fused variant of tc_decode_partial_out + all-gather + tc_combine_partials for the ranks of one
 * node (one process per GPU, every GPU a peer of every other over NVLink); no counterpart in the
 * reference. One launch per rank: the CTA that finishes a (batch, KV head) unit stores this rank's
 * partial O and LSE into every rank's exchange block with plain peer stores, every 4-byte value
 * paired with the call's epoch in one aligned 8-byte word, then polls its own block (bounded: 2 s,
 * then tc_device_status != 0) until the words of every rank carry that epoch, and merges the `world`
 * partials with the arithmetic of tc_combine_partials. No fence or separate flag sits between a
 * store and its remote read. Every rank ends with the full result in out (BF16 [B,1,Hq,128]) and lse
 * (fp32 [B,Hq]). peer_blocks[r] is rank r's exchange block as mapped into this process
 * (peer_blocks[rank] is this rank's own block). All ranks must make the same sequence of calls with
 * the same batch, kv_heads and world on the same blocks. peer_block_size is the size in bytes every one of
 * those blocks was created with; a call whose (batch, kv_heads, world) needs more than that is rejected,
 * because its stores would leave the blocks on the other GPUs. splits * Hkv * B CTAs must be resident at
 * once (rejected otherwise). Plain stores only; no collective library call is involved.
 *
 * Exchange blocks: tc_peer_block_bytes gives the size for (batch, kv_heads, world);
 * tc_peer_block_create allocates and zeroes one on `device` and returns a 64-byte interprocess handle;
 * the other ranks map it with tc_peer_block_open (never the creating process itself) and unmap it
 * with tc_peer_block_close; the owner frees it with tc_peer_block_destroy after everyone unmapped. */
int tc_decode_exchange_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                           const void* vnew, const int32_t* old_lengths, void* out, float* lse, float* workspace_o,
                           int64_t workspace_o_elems, float* workspace_lse, int64_t workspace_lse_elems, int64_t batch,
                           int64_t capacity, int64_t kv_heads, int64_t num_splits, int64_t mapping, int append,
                           int64_t kv_shard_start, int64_t world, int64_t rank, void* const* peer_blocks,
                           int64_t peer_block_size);
int tc_peer_block_bytes(int64_t batch, int64_t kv_heads, int64_t world, int64_t* bytes);
int tc_peer_block_create(int device, int64_t bytes, void** block, unsigned char* handle64);
int tc_peer_block_open(int device, const unsigned char* handle64, void** block);
int tc_peer_block_close(int device, void* block);
int tc_peer_block_destroy(int device, void* block);

/* Replaces `resources(q,kcache,old_lengths,num_splits,mapping,append) -> int[]`
 * (decode.cu:203-229): 12 header values, 8 attributes of the split kernel, 8 of the standalone
 * combine kernel, 6 tail values. */
int tc_decode_resources(int device, int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits,
                        int64_t mapping, int append, int64_t* values, int64_t capacity_values, int64_t* count);

/* ---------------------------------------------------------------------------------- the step before decode
 * Fused QKV projection + per-head RMS norm + RoPE for one new token per sequence, writing q, knew and vnew in
 * the layout tc_decode_forward_out takes. No counterpart in the reference, whose decode kernel is handed
 * pre-rotated Q/K and one new row (ab_fused_splitkv.cuh:189).
 *   x BF16 [tokens, hidden] (1 <= tokens <= 8, hidden a multiple of 64); w_qkv BF16 [(q_heads + 2*kv_heads)*128,
 *   hidden] row-major, rows ordered q heads, k heads, v heads; y = x w_qkv^T accumulated in FP32.
 *   q_norm_weight / k_norm_weight BF16 [128] or NULL: y * rsqrt(mean(y^2) + rms_eps) rounded to BF16, times the
 *   weight, rounded to BF16 (Qwen3's per-head norm). Without a weight y is rounded to BF16.
 *   rope_cos / rope_sin FP32 [rope_positions, 64] or both NULL, positions int32 [tokens] on the device
 *   (old_lengths): rotate-half RoPE of the q and k heads as in tc_decode_rope_forward_out. v heads get neither
 *   norm nor RoPE.
 *   q_out BF16 [tokens,1,q_heads,128], knew_out / vnew_out BF16 [tokens,1,kv_heads,128].
 * Weight-streaming, HBM-bound: one cluster of up to 4 CTAs per head splits the hidden dimension and reduces
 * through distributed shared memory. The kernel is launched with programmatic dependent launch and starts
 * reading w_qkv before the preceding kernel of the stream has finished: the weights must not be an output of
 * that kernel (x, positions, tables and norm weights may be). */
int tc_qkv_rope_forward_out(int device, void* stream, const void* x, const void* w_qkv, const void* q_norm_weight,
                            const void* k_norm_weight, const float* rope_cos, const float* rope_sin,
                            int64_t rope_positions, const int32_t* positions, void* q_out, void* knew_out,
                            void* vnew_out, int64_t tokens, int64_t hidden, int64_t q_heads, int64_t kv_heads,
                            double rms_eps);

/* The same call with options. TC_PROJECT_RELEASE_EARLY: by default the kernel launched after this one (if it is a
 * programmatic dependent launch) may begin once this kernel has seen its own stream dependency resolve, so whatever
 * that follower does ahead of its own dependency overlaps this kernel only. With the flag the follower is released
 * at once and may also overlap the kernel launched BEFORE this one: the caller promises that the follower's
 * independent part is safe beside that kernel too (always true when the follower is another projection, which
 * reads only its weights ahead of its dependency; for a decode step launched with a cache promise the promise must
 * then hold for both predecessors). Results are unchanged; a chain of projections runs about 10 % faster. */
#define TC_PROJECT_RELEASE_EARLY 1
int tc_qkv_rope_forward_out_flags(int device, void* stream, const void* x, const void* w_qkv,
                                  const void* q_norm_weight, const void* k_norm_weight, const float* rope_cos,
                                  const float* rope_sin, int64_t rope_positions, const int32_t* positions, void* q_out,
                                  void* knew_out, void* vnew_out, int64_t tokens, int64_t hidden, int64_t q_heads,
                                  int64_t kv_heads, double rms_eps, int flags);

/* ---------------------------------------------------------------------------------- two-tile exchange
 * Complete attention for 64 queries x 64 keys per (batch, head), D = 128, FP16 or BF16, generated as
 * straight-line code from a residency-exchange plan. Replaces `forward_out(q,k,v,out!,lse!,nonce,causal,
 * nonce_is_zero,diagnostic_non_nan_asserted)` and `resources(q,causal) -> int[14]`
 * (tilecadence/cuda/exchange/binding.cpp:32-72, schemas :79-81). q/k/v/out contiguous [B,64,H,128],
 * lse fp32 [B,H,64]. The nonce arguments of the reference exist only for its opaque-recovery mode,
 * which these plans never use. resources: block_m, block_n, head_dim, value_stripe_dim, threads,
 * dynamic smem, static smem, registers/thread, local bytes/thread, binary version, PTX version,
 * active CTAs/SM, required nonce elements (0), diagnostic guard (0). */
int tc_exchange_forward_out(int device, void* stream, const void* q, const void* k, const void* v, void* out,
                            float* lse, int64_t batch, int64_t heads, int dtype_fp16, int causal);
int tc_exchange_resources(int device, int dtype_fp16, int causal, int64_t values[14]);

#ifdef __cplusplus
}
#endif
#endif /* TILECADENCE_B200_H */
