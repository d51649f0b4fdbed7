/*
 * phasekv_b200 — C ABI of the B200 (sm_100a) implementation of PhaseKV's stage-B hot path:
 * sub-byte quantise+pack, the three-tier split-K decode attention and its log-sum-exp merge.
 *
 * The reference has no FFI of its own: its boundary is a set of Python callables
 * (src/phasekv/kernels/packing.py, attention_triton.py, launch_config.py).  Each entry
 * point below names the reference function it stands behind.  Conventions:
 *   - every pointer is a DEVICE pointer unless its comment says "host";
 *   - float16 data is passed as `const void*` / `void*` (IEEE binary16, little endian);
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*), nothing synchronises;
 *   - nothing is allocated and no pointer is retained after the call returns;
 *   - the return value is 0 on success or a negative PKV_E_* code; pkv_strerror() names it.
 */
#ifndef PHASEKV_B200_H
#define PHASEKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PKV_OK 0
#define PKV_E_BITS (-1)      /* bit width not in {2, 4, 8} */
#define PKV_E_SHAPE (-2)     /* negative / zero / inconsistent sizes */
#define PKV_E_NULL (-3)      /* required pointer is NULL */
#define PKV_E_LAYOUT (-4)    /* segment kind / group size not supported by the kernels */
#define PKV_E_WORKSPACE (-5) /* scratch buffer too small */
#define PKV_E_CUDA (-6)      /* a CUDA runtime call failed; see pkv_last_cuda_error() */
#define PKV_E_LIMIT (-7)     /* a documented maximum was exceeded */

typedef void* pkv_stream_t; /* cudaStream_t */

int pkv_abi_version(void);
const char* pkv_strerror(int code);
/* cudaError_t value of the last failing CUDA call made by this library on the calling thread. */
int pkv_last_cuda_error(void);
/* attention_triton.py:599-601 (_device_sm_count) */
int pkv_device_sm_count(int device, int* sm_count /* host */);

/* ---------------------------------------------------------------- packing ---------- */

/* packing.py:41-65 pack_low_bits: codes u8 [rows, len] -> out u8 [rows, ceil(len / (8/bits))];
 * code i of a byte sits at bits [i*bits, (i+1)*bits); unused tail bits are zero. */
int pkv_pack_low_bits(const uint8_t* codes, int64_t rows, int64_t len, int bits, uint8_t* out,
                      pkv_stream_t stream);

/* packing.py:67-79 unpack_low_bits: packed u8 [rows, row_bytes] -> out u8 [rows, len],
 * len <= row_bytes * (8/bits). */
int pkv_unpack_low_bits(const uint8_t* packed, int64_t rows, int64_t row_bytes, int64_t len,
                        int bits, uint8_t* out, pkv_stream_t stream);

/* packing.py:115-155 quantize_pack.  x is float16 viewed as [outer, axis_len, inner]; groups of
 * `group` (1 <= group <= axis_len, already clamped as packing.py:130 does) run along axis_len.
 * Outputs carry the axis last:  packed u8 [outer, inner, ceil(axis_len / (8/bits))],
 * scale and mins float16 [outer, inner, ceil(axis_len / group)].
 * K of a KV cache is (outer = B*Hkv, axis_len = S, inner = hd); V is (outer = B*Hkv*S,
 * axis_len = hd, inner = 1). Codes, scales and zeros are bit-identical to the reference on CPU. */
int pkv_quantize_pack(const void* x, int64_t outer, int64_t axis_len, int64_t inner, int bits,
                      int64_t group, uint8_t* packed, void* scale, void* mins, pkv_stream_t stream);

/* The same with padded output rows: consecutive rows of `packed` are packed_pitch bytes apart and rows of
 * scale / mins meta_pitch elements apart (0 = dense, as above; otherwise >= the dense row length).  The
 * padding is not written.  A key tensor whose rows are padded to whole 64-token tiles
 * (packed_pitch = ceil(S/64) * 64 * bits / 8, meta_pitch a multiple of 8 and >= 2 * ceil(S/64)) lets the
 * decode kernel stream a segment of ANY length with 16-byte copies; with dense rows that holds only for
 * S % 64 == 0 and other lengths take a slower loader.  The reference's PackedTensor stays valid: its
 * `packed`, `scale`, `mins` tensors become views with a row stride. */
int pkv_quantize_pack_pitched(const void* x, int64_t outer, int64_t axis_len, int64_t inner, int bits,
                              int64_t group, uint8_t* packed, void* scale, void* mins, int64_t packed_pitch,
                              int64_t meta_pitch, pkv_stream_t stream);

/* packing.py:158-175 unpack_dequantize: inverse of the above, out float16 [outer, axis_len, inner],
 * computed as float32 code*scale then +mins (two roundings) then rounded to float16. */
int pkv_unpack_dequantize(const uint8_t* packed, const void* scale, const void* mins, int64_t outer,
                          int64_t axis_len, int64_t inner, int bits, int64_t group, void* out,
                          pkv_stream_t stream);

/* ---------------------------------------------------------------- decode ----------- */

/* One stretch of cached tokens of one layer, all KV heads.  Three layouts: */
#define PKV_SEG_KIVI 0     /* K packed along tokens:  k_packed u8 [Hkv, hd, ceil(S/kvpb)], k_scale/k_mins f16 [Hkv, hd, ceil(S/k_group)]
                              V packed along dims:    v_packed u8 [Hkv, S, ceil(hd/vvpb)], v_scale/v_mins f16 [Hkv, S, ceil(hd/v_group)]
                              (LayerTiers.prompt / prompt_extensions / cold, phasekv_cache.py:101-107) */
#define PKV_SEG_PER_TOKEN 1 /* K and V both packed along dims (quantize_pack(x, bits, -1, gs) of [Hkv, S, hd]):
                              *_packed u8 [Hkv, S, ceil(hd/vpb)], *_scale/_mins f16 [Hkv, S, ceil(hd/group)]
                              (attention_triton.py:95-142, the published micro-benchmark layout) */
#define PKV_SEG_FP16 2     /* k_packed / v_packed point at float16 [Hkv, >=S, hd] with `head_stride` elements
                              between heads (LayerTiers.hot_views(), phasekv_cache.py:75-79) */

typedef struct pkv_segment {
    const void* k_packed;
    const void* k_scale;
    const void* k_mins;
    const void* v_packed;
    const void* v_scale;
    const void* v_mins;
    int64_t seq_len;     /* S: tokens in this segment (> 0) */
    int64_t head_stride; /* PKV_SEG_FP16: elements between consecutive KV heads.  PKV_SEG_KIVI: token rows between
                            consecutive KV heads of v_packed / v_scale / v_mins (0 = seq_len, i.e. dense) */
    int32_t kind;        /* PKV_SEG_* */
    int32_t k_bits, v_bits;   /* 2, 4 or 8 (ignored for PKV_SEG_FP16) */
    int32_t k_group, v_group; /* quantisation group sizes (after clamping to the axis length) */
    int32_t num_splits;       /* 0 = let the library choose; else as plan_kivi_decode(num_splits=...) */
    /* PKV_SEG_KIVI only; 0 = dense.  Bytes between consecutive channel rows of k_packed, and elements between
     * consecutive rows of k_scale / k_mins (see pkv_quantize_pack_pitched).  Heads are hd rows apart. */
    int64_t k_row_pitch;
    int64_t k_meta_pitch;
    int32_t flags;    /* PKV_SEG_FLAG_* */
    /* PKV_SEG_KIVI only; 0 = every token counts.  Otherwise the segment is a run of equal slots of slot_tokens
     * tokens (32 or 64) of which only the first slot_valid hold tokens; the rest of a slot is padding that the
     * kernels mask out.  This is how a run of small cold segments (one per cooling step, each quantised on its own)
     * is presented as ONE segment: every step's tokens sit at the start of a slot whose key group is the step's
     * own group (see pkv_cold_select_pack_layers). */
    int16_t slot_tokens;
    int16_t slot_valid;
    /* PKV_SEG_FP16 and PKV_SEG_KIVI; NULL = seq_len is the length.  Otherwise a DEVICE address of an int32 holding
     * the number of tokens that count, read when the kernel runs (after everything earlier in the stream):
     * min(seq_len, *seq_len_dev) tokens are attended to, and seq_len is the CAPACITY the launch is sized for.  This
     * keeps a captured CUDA graph of decode calls valid while the float16 tier (or a run of cold slots) grows: the
     * owner of the cache updates the int32 in stream order instead of re-describing the segment. */
    const int32_t* seq_len_dev;
} pkv_segment_t;

/* The packed tensors of this segment may have been written by the kernel that was launched on `stream` directly
 * before this decode call (pkv_quantize_pack*, pkv_cold_select_pack, a copy).  Decode launches are programmatic
 * dependents of the previous kernel of the stream and begin to fetch packed segments before that kernel's
 * writes are guaranteed visible; with this flag the segment is read only after the dependency is resolved.
 * Segments written by anything earlier in the stream need no flag. */
#define PKV_SEG_FLAG_FRESH 1

#define PKV_MAX_SEGMENTS 4096

/* Scratch bytes pkv_decode_attention needs for these segments (host array). */
int pkv_decode_workspace_bytes(const pkv_segment_t* segs /* host */, int n_segs, int num_q_heads,
                               int num_kv_heads, int head_dim, int sm_count, size_t* bytes /* host */);

/* Kernel launches pkv_decode_attention makes for these segments: the split-K launches (one per 24 segments a
 * kernel takes; normally one) plus one merge launch.  No counterpart in the
 * reference, which launches one kernel and a handful of torch ops per segment (attention_triton.py:643-669). */
int pkv_decode_launches(const pkv_segment_t* segs /* host */, int n_segs, int num_q_heads, int num_kv_heads,
                        int head_dim, int sm_count, int* launches /* host */);

/* attention_triton.py:643-669 fused_phasekv_decode (and :604-639 _kivi_layer_partial, :285-297
 * _fp16_layer_partial, :487-511 fused_three_tier_decode, :95-142 / :269-276 decode_attention_packed[_splitk]):
 * single-query attention of q float16 [Hq, hd] over the concatenation of `segs`, without ever
 * writing dequantised K/V to memory.  One split-K launch covers all segments (more than 24 segments, or
 * segments that only the layout-generic kernel takes, add launches), one merge launch follows.
 * Which kernel serves a segment: with head_dim 128, a GQA group of at most 8, 16-byte aligned buffers, equal
 * K and V widths and groups of 32, PKV_SEG_KIVI and PKV_SEG_FP16 segments go to the tensor-core kernel, and so do
 * PKV_SEG_PER_TOKEN segments (a kernel of their own) unless the same call also holds a PKV_SEG_KIVI segment;
 * everything else goes to the general kernel (any head_dim <= 256 that is a multiple of 4, any group sizes,
 * different K and V widths).  The result does not depend on the route beyond rounding.
 * Outputs (each may be NULL):
 *   out  float16 [Hq, hd]  = acc / l
 *   m, l float32 [Hq], acc float32 [Hq, hd]: the un-normalised partial of attention_triton.py:257-266,
 *   mergeable across segments, layers of a tier, or GPUs with pkv_merge_partials.
 * `workspace` is device scratch of at least pkv_decode_workspace_bytes() (16-byte aligned; its contents need
 * no initialisation); calls that share it must not overlap on the GPU. */
int pkv_decode_attention(const void* q, const pkv_segment_t* segs /* host */, int n_segs,
                         int num_q_heads, int num_kv_heads, int head_dim, float sm_scale,
                         int sm_count, void* workspace, size_t workspace_bytes, void* out, float* m,
                         float* l, float* acc, pkv_stream_t stream);

/* No counterpart in the reference.  Same computation and outputs as pkv_decode_attention, for callers that
 * cannot hand over scratch memory because they may not allocate on the device (a plugin with a fixed memory
 * budget, code running under stream capture).  The split-K partials go to an array of
 * PKV_STATIC_SCRATCH_BYTES that is part of the library image on every GPU that loads it.  Requests that need
 * more scratch than that fail with PKV_E_LIMIT.  The first call on each device looks the array's device address
 * up (make that call before starting a stream capture).  All calls on a device share the array: calls whose
 * kernels may overlap on the GPU must not use this entry point concurrently.  No device memory is allocated
 * or freed. */
#define PKV_STATIC_SCRATCH_BYTES (8u << 20)
int pkv_decode_attention_static(const void* q, const pkv_segment_t* segs /* host */, int n_segs,
                                int num_q_heads, int num_kv_heads, int head_dim, float sm_scale, int sm_count,
                                void* out, float* m, float* l, float* acc, pkv_stream_t stream);

/* Batched decode for serving: `batch` independent sequences, each with its own list of segments, attended in
 * ONE split-K launch and ONE merge launch.  The reference's entry point is batch 1 only
 * (attention_triton.py:655-657: fused_phasekv_decode raises unless orig_shape[0] == 1) and a batch is served by
 * looping it; this pair of calls is what such a loop is replaced by.
 *
 * pkv_decode_batch_plan (host only, no CUDA call): sequence i owns segs[seg_offsets[i] .. seg_offsets[i+1]).
 * It cuts every segment into work items of balanced cost, orders them longest first, and writes a
 * position-independent table (segment descriptors, work list, per-sequence ranges of partials) into `table`
 * (host memory, 16-byte aligned).  `table_bytes` receives the bytes used, `workspace_bytes` the device scratch
 * the launch needs.  With table == NULL only the two sizes are computed.  Every segment must be one the
 * tensor-core kernel takes (KIVI layout with head_dim 128, group 32, equal K/V bits, or float16, not the per-token layout; GQA group
 * <= 8; 16-byte aligned buffers), otherwise PKV_E_LAYOUT: serve such sequences one by one.
 * PKV_E_WORKSPACE when table_capacity is too small.  The plan depends on lengths and pointers only, so it
 * stays valid until one of them changes.
 *
 * pkv_decode_attention_batched: q float16 [batch, Hq, hd], out float16 [batch, Hq, hd].  `table_device` is a
 * copy of the table in device memory made by the caller (any stream-ordered copy before this call);
 * `table_host` is the host original, read for the launch geometry only.  Same workspace rules as
 * pkv_decode_attention. */
int pkv_decode_batch_plan(const pkv_segment_t* segs /* host */, const int32_t* seg_offsets /* host [batch+1] */,
                          int batch, int num_q_heads, int num_kv_heads, int head_dim, int sm_count,
                          void* table /* host, may be NULL */, size_t table_capacity, size_t* table_bytes,
                          size_t* workspace_bytes);
int pkv_decode_attention_batched(const void* q, const void* table_host, const void* table_device,
                                 float sm_scale, void* workspace, size_t workspace_bytes, void* out,
                                 pkv_stream_t stream);

/* A chunk of new prompt tokens in one launch pair.  The reference attends to a chunk of N input tokens with N
 * consecutive single-query calls, each after appending that token's K/V (qwen2_attention.py:99-106: "write one,
 * compute one"), so that no query sees a later token of its chunk.  Here all N tokens are written to the
 * float16 tier first and the causal rule is applied by length: `segs` describes the layer as for
 * pkv_decode_attention, its LAST segment being the float16 tier INCLUDING the N new tokens at its end; query i
 * (0-based) attends to all other segments in full and to the first seq_len - (N - 1 - i) float16 tokens.
 * The plan is a pkv_decode_batch_plan table with one entry per query: run it with
 * pkv_decode_attention_batched on q float16 [N, Hq, hd] -> out float16 [N, Hq, hd].  Same layout rules and
 * errors as pkv_decode_batch_plan; PKV_E_SHAPE if the last segment is not float16 or shorter than the chunk. */
int pkv_decode_chunk_plan(const pkv_segment_t* segs /* host */, int n_segments, int chunk_len, int num_q_heads,
                          int num_kv_heads, int head_dim, int sm_count, void* table /* host, may be NULL */,
                          size_t table_capacity, size_t* table_bytes, size_t* workspace_bytes);

/* attention_triton.py:257-266 _reduce_splits and :300-307 _merge_partials:
 * m, l float32 [n_parts, Hq] and acc float32 [n_parts, Hq, hd] (contiguous) are combined with
 * M = max m, w = exp(m - M), L = sum w*l, A = sum w*acc.  out float16 [Hq, hd] = A / L;
 * m_out/l_out/acc_out (optional) receive (M, L, A). */
int pkv_merge_partials(const float* m, const float* l, const float* acc, int n_parts, int num_q_heads,
                       int head_dim, void* out, float* m_out, float* l_out, float* acc_out,
                       pkv_stream_t stream);

/* The same merge over partials that are not packed densely: partial p has its m and l rows ml_stride floats
 * after those of partial p-1 and its acc rows acc_stride floats after (ml_stride >= Hq, acc_stride >= Hq*hd,
 * acc_stride % 4 == 0).  This is the layout an all-gather of one flat per-rank message
 * [acc Hq*hd | m Hq | l Hq] leaves behind (both strides Hq*(hd+2)): the sequence-sharded decode merges the
 * ranks' partials in place, without repacking. */
int pkv_merge_partials_strided(const float* m, const float* l, const float* acc, int n_parts, int64_t ml_stride,
                               int64_t acc_stride, int num_q_heads, int head_dim, void* out, float* m_out,
                               float* l_out, float* acc_out, pkv_stream_t stream);

/* ---------------------------------------------------------------- multi-GPU ------- */

/* Sequence-sharded decode (long context, batch 1) without a collective library: no counterpart in the
 * reference, which is single-GPU; the merge algebra is attention_triton.py:257-266, 300-307 across GPUs.
 * Every rank (one process per GPU of one node) holds a contiguous shard of the prompt tier (one rank also the
 * cold and hot tiers).  A call is one split-K launch over the local segments plus ONE kernel that merges the
 * local partials, stores the result into every peer's exchange buffer over NVLink (plain peer stores into
 * memory mapped with CUDA IPC), publishes an epoch flag, waits for the peers' rows to arrive in its OWN buffer
 * and merges them; every rank ends with the full out [Hq, hd].  The wait is bounded by a number of polling
 * passes and by the clock: when it runs out the kernel sets a status word, writes NaN to its output rows and
 * returns (read the word with pkv_exchange_status).  The failure is sticky: ranks that missed each other once
 * are out of step for good, so every later call on that exchange returns NaN rows at once, without pushing
 * or waiting; destroy the exchange and build a new one.
 *
 * Set-up (allocates; not for the request path): pkv_exchange_create allocates this rank's buffer on the current
 * device and returns a 64-byte IPC handle; the caller gathers the handles of all ranks in rank order (any host
 * transport) and passes the world*64 bytes to pkv_exchange_connect.  All ranks must make the same sequence of
 * pkv_decode_attention_sharded calls on an exchange; calls on one exchange must not overlap on the GPU.
 * pkv_exchange_connect_loopback maps every peer slot onto the local buffer (single-process testing: with
 * world 1 it is a complete exchange, with world > 1 the peers never arrive and the bounded wait runs out). */
typedef struct pkv_exchange pkv_exchange_t;
#define PKV_IPC_HANDLE_BYTES 64
#define PKV_MAX_WORLD 16
int pkv_exchange_create(int world, int rank, int num_q_heads, int head_dim, pkv_exchange_t** ex /* host */,
                        void* handle_out /* host, 64 bytes */);
int pkv_exchange_connect(pkv_exchange_t* ex, const void* handles /* host, world * 64 bytes */);
int pkv_exchange_connect_loopback(pkv_exchange_t* ex);
int pkv_exchange_set_spin_limit(pkv_exchange_t* ex, unsigned polls);
/* Most microseconds one wait may take (default 250 000).  A wait ends at whichever bound it meets first.  Ranks
 * whose set-up takes different times meet at a host barrier before their first call. */
int pkv_exchange_set_wait_us(pkv_exchange_t* ex, unsigned microseconds);
int pkv_exchange_status(pkv_exchange_t* ex, int* timed_out /* host; synchronises */);
int pkv_exchange_destroy(pkv_exchange_t* ex);
/* n_segs may be 0 (a rank without tokens contributes the neutral partial; q, segs, workspace are then unused). */
int pkv_decode_attention_sharded(const void* q, const pkv_segment_t* segs /* host */, int n_segs,
                                 int num_q_heads, int num_kv_heads, int head_dim, float sm_scale, int sm_count,
                                 void* workspace, size_t workspace_bytes, pkv_exchange_t* ex, void* out,
                                 pkv_stream_t stream);

/* ---------------------------------------------------------------- cold tier -------- */

/* phasekv_cache.py:322-340 _cool_aged_tokens for one layer: among the oldest `aged` tokens of the
 * hot buffers hot_k/hot_v float16 [rows, capacity, hd] (rows = B*Hkv), keep the `keep` tokens with the
 * largest value L2 norm per row (ascending position order; all of them when keep == aged), quantise and
 * pack them (K along tokens, V along dims, `bits`, `group`), and move the remaining hot_len - aged tokens
 * to the start of the hot buffers.
 *   k_packed u8 [rows, hd, ceil(keep/vpb)], k_scale/k_mins f16 [rows, hd, ceil(keep/min(group,keep))]
 *   v_packed u8 [rows, keep, ceil(hd/vpb)], v_scale/v_mins f16 [rows, keep, ceil(hd/min(group,hd))]
 *   indices int64 [rows, keep] (optional): the kept positions. */
int pkv_cold_select_pack(void* hot_k, void* hot_v, int64_t rows, int64_t capacity, int head_dim,
                         int64_t hot_len, int64_t aged, int64_t keep, int bits, int64_t group,
                         uint8_t* k_packed, void* k_scale, void* k_mins, uint8_t* v_packed,
                         void* v_scale, void* v_mins, int64_t* indices, pkv_stream_t stream);

/* The same for every layer of a model in ONE launch, writing into pre-allocated arenas (no counterpart in the
 * reference, which cools layer by layer with ~50 torch launches each, phasekv_cache.py:322-340).  `layers` is a
 * DEVICE array of n_layers entries holding each layer's hot buffers and the BASE pointers of its outputs (it stays
 * valid across calls while the buffers do); all layers share rows, capacity, hot_len, aged, keep.  The outputs of
 * this call start slot_k_bytes bytes into every row of k_packed, slot_k_groups elements into every row of
 * k_scale / k_mins, and slot_v_tokens token rows into every (batch, head) block of the value outputs; rows of
 * k_packed are k_row_pitch bytes apart, rows of k_scale / k_mins k_meta_pitch elements, (batch, head) blocks of the
 * value outputs v_row_tokens token rows.  With slots of ceil(keep / group) * group tokens, zero-initialised arenas
 * and one group per `group` tokens, the arena of a layer is one PKV_SEG_KIVI segment with slot_tokens / slot_valid
 * set, and each step's part of it is bit-identical to what pkv_cold_select_pack writes into tensors of its own. */
typedef struct pkv_cold_layer {
    void* hot_k;
    void* hot_v;
    uint8_t* k_packed;
    void* k_scale;
    void* k_mins;
    uint8_t* v_packed;
    void* v_scale;
    void* v_mins;
    int64_t* indices; /* [rows, keep] of this call, may be NULL */
} pkv_cold_layer_t;
int pkv_cold_select_pack_layers(const pkv_cold_layer_t* layers /* device */, int n_layers, int64_t rows,
                                int64_t capacity, int head_dim, int64_t hot_len, int64_t aged, int64_t keep,
                                int bits, int64_t group, int64_t k_row_pitch, int64_t k_meta_pitch,
                                int64_t v_row_tokens, int64_t slot_k_bytes, int64_t slot_k_groups,
                                int64_t slot_v_tokens, pkv_stream_t stream);

/* ---------------------------------------------------------------- stage A (dense cache) -------- */

#define PKV_DTYPE_F16 0
#define PKV_DTYPE_BF16 1
#define PKV_DTYPE_F32 2

/* quant.py:34-79 _grouped_affine_quant_dequant (behind quantize_key :82-91, quantize_value :94-101, used in
 * place on cache slices by prompt_tier.py:107-118 and decode_tier.py:78-88): x viewed as [outer, axis_len, inner]
 * with `outer_stride` elements between outer indices (0 = dense; larger for a token slice of a longer cache),
 * groups of `group` (clamped to axis_len by the caller) along axis_len, float32 scale = max(max-min, 1e-8)/qmax
 * and zero = min, out = round((x-min)/scale).clamp(0, qmax) * scale + min rounded to the element type.
 * bits 1..15 (>= 16 is the caller's no-op).  out may equal x.  Bit-identical to the reference on a CPU. */
int pkv_fake_quant(const void* x, void* out, int dtype, int64_t outer, int64_t axis_len, int64_t inner,
                   int64_t outer_stride, int bits, int64_t group, pkv_stream_t stream);

/* hetero_cache.py:98-113 value_norm_signal: out float32 [rows, n_tokens] = L2 norm over head_dim of the first
 * n_tokens tokens of each row of v [rows, >= n_tokens, head_dim] (`row_stride` elements between rows). */
int pkv_value_norm(const void* v, int dtype, int64_t rows, int64_t row_stride, int64_t n_tokens, int head_dim,
                   float* out, pkv_stream_t stream);

/* hetero_cache.py:157-167 topk_per_head followed by the ascending sort every consumer applies
 * (hetero_cache.py:146, phasekv_cache.py:332): indices int64 [rows, keep] = positions of the `keep` largest
 * entries of each row of signal float32 [rows, n], NaN largest (as torch.topk orders it), ties to the lower
 * position.  Rows of up to 4096 entries are ranked by counting, longer rows by a radix select. */
int pkv_topk_rows(const float* signal, int64_t rows, int64_t n, int64_t keep, int64_t* indices, pkv_stream_t stream);

/* hetero_cache.py:120-154 evict_per_head / phasekv_cache.py:110-114 _gather_kv for one tensor:
 * dst [rows, keep, token_bytes] = src [rows, src_tokens, token_bytes] gathered at indices int64 [rows, keep].
 * token_bytes % 16 == 0, 16-byte aligned buffers. */
int pkv_gather_tokens(const void* src, void* dst, const int64_t* indices, int64_t rows, int64_t src_tokens,
                      int64_t keep, int64_t token_bytes, pkv_stream_t stream);

/* ---------------------------------------------------------------- model adapter ------- */

/* qwen2_attention.py:79-106 (and examples/llama_phasekv_adapter.py:63-85) between the projections and decode
 * attention, for n_tokens new tokens of one layer (batch 1) in one launch: apply_rotary_pos_emb to q and k, the
 * .to(float16) of q, k and v, and the write of k and v into the float16 tier (append_hot / append_prompt_token).
 *   q [n_tokens, Hq, hd], k and v [n_tokens, Hkv, hd] of `dtype` (PKV_DTYPE_F16 / PKV_DTYPE_BF16), with
 *   *_token_stride elements between consecutive tokens (the projections' row pitch);
 *   cos, sin [n_tokens, hd] of `rope_dtype` (any PKV_DTYPE_*), rope_token_stride elements between tokens: the
 *   full-width tables transformers builds (both halves filled);
 *   q_out float16 [n_tokens, Hq, hd] dense; hot_k / hot_v float16 [Hkv, capacity, hd]: token i goes to slot
 *   `slot` + i.
 * Rounded as torch rounds when the rotation runs in `dtype`: x*cos, rotate_half(x)*sin and their sum are each
 * rounded to `dtype`, then converted to float16.
 * slot_dev (optional, DEVICE int32): when given, the first slot is *slot_dev + slot, read when the kernel runs, so
 * that a captured graph keeps appending behind a growing tier; a slot outside [0, capacity - n_tokens] writes
 * nothing to the tier (the rotated queries are still produced). */
int pkv_rope_append(const void* q, const void* k, const void* v, int dtype, int64_t q_token_stride,
                    int64_t k_token_stride, int64_t v_token_stride, const void* cos, const void* sin,
                    int rope_dtype, int64_t rope_token_stride, int n_tokens, int num_q_heads, int num_kv_heads,
                    int head_dim, void* q_out, void* hot_k, void* hot_v, int64_t capacity, int64_t slot,
                    const int32_t* slot_dev, pkv_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PHASEKV_B200_H */
