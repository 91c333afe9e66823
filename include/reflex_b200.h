/*
 * reflex_b200.h -- C ABI of libreflex_b200.so: the paged-KV attention path of
 * reflex-infer's Python kernel library, as hand-written sm_100a CUDA kernels.
 *
 * Conventions (they follow the reference's own C++ API, include/reflex/infer.h:16-23,
 * 92,189-220, and its API principles, docs/library-architecture.md:57-64,100-105):
 *   - every entry point takes one pointer to a plain args struct and returns an int
 *     status; the first six codes are the reference's `Status` values in its order;
 *   - all pointers are raw DEVICE pointers unless a field says "host";
 *   - the library never allocates, frees or synchronises: outputs and workspaces are
 *     caller-owned, every kernel is enqueued on `stream` (a cudaStream_t, 0 = default);
 *   - strides are in ELEMENTS; index tensors are int64 (slots, block tables) and int32
 *     (context lengths, positions) exactly as in the reference
 *     (kernels/kv_cache/triton_kv_paged.py:9-15);
 *   - nothing throws, aborts or traps; invalid arguments come back as
 *     RFX_INVALID_ARGUMENT with a message in rfx_last_error().
 *
 * Paged cache layout (kernels/kv_cache/triton_kv_paged.py:9-15):
 *   k_cache, v_cache : [num_blocks, num_kv_heads, block_size, head_dim]
 *   slot             = page * block_size + position_in_page
 *   block_table[b,j] = physical page of logical block j of request b
 *
 * int8 KV with one fp32 scale per (position, kv head) -- the reference's `kv_int8` with
 * `k_scales[kv_pos * n_kv_heads + kv_head]` (src/kernels/attention.cu:91-96,141-150;
 * include/reflex/infer.h:189-203), carried over to pages:
 *   k_cache, v_cache : int8 [num_blocks, num_kv_heads, block_size, head_dim]
 *   k_scales, v_scales : fp32 [num_blocks, num_kv_heads, block_size]
 *   value = int8 * scale. The writer (rfx_rope_append with kv_int8) quantises each row with
 *   scale = max|x| / 127 (1 for an all-zero row) and q = round-half-even(x / scale), in fp32.
 */
#ifndef REFLEX_B200_H_
#define REFLEX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RFX_ABI_VERSION 2

/* include/reflex/infer.h:16-23 (first six, same order) + three additions. */
typedef enum {
    RFX_SUCCESS = 0,
    RFX_UNSUPPORTED_DEVICE = 1,
    RFX_UNSUPPORTED_MODEL = 2,
    RFX_UNSUPPORTED_QUANT_FORMAT = 3,
    RFX_INVALID_ARGUMENT = 4,
    RFX_NOT_IMPLEMENTED = 5,
    RFX_CUDA_ERROR = 6,          /* a CUDA runtime/driver call failed; see rfx_last_error() */
    RFX_TIMEOUT = 7,             /* a bounded device-side wait expired (status word) */
    RFX_WORKSPACE_TOO_SMALL = 8
} rfx_status;

typedef enum { RFX_F32 = 0, RFX_BF16 = 1, RFX_F16 = 2 } rfx_dtype;

typedef void* rfx_stream; /* cudaStream_t; mirrors StreamHandle, include/reflex/infer.h:92 */

int rfx_abi_version(void);
/* sizeof() of the args struct with the given index (0 RfxKvAppendArgs, 1 RfxKvLookupArgs,
 * 2 RfxRopeArgs, 3 RfxRopeTableArgs, 4 RfxRopeAppendArgs, 5 RfxSoftmaxArgs,
 * 6 RfxAttentionArgs, 7 RfxPagedAttentionArgs, 8 RfxCombineArgs, 9 RfxHeadGatherArgs,
 * 10 RfxPeerHandle, 11 RfxLinearNormArgs; 0 for anything else), so
 * a foreign-function binding can verify its struct mirrors before the first call. */
size_t rfx_args_size(int which);
const char* rfx_status_string(int status);
/* Thread-local text of the last non-success status returned on this host thread. */
const char* rfx_last_error(void);
/* Debug switches (tests, cross-checks; no counterpart in the reference). The library reads the
 * environment variable REFLEX_B200_DEBUG once, as comma-separated words:
 *   no_tc            scalar kernels where a tcgen05 kernel would run (attention, linear + norm)
 *   prefill_nosplit  chunked prefill is not split over the keys
 *   mixed=1 / mixed=0  one-row requests of a split batch always / never go to the decode kernel
 *                    (default: they do whenever that kernel takes the shapes)
 *   tma2d            the decode kernel's 2-D tensor maps
 * rfx_debug_set_flags(words) replaces them for the whole process (NULL: back to the environment's). */
int rfx_debug_set_flags(const char* words);

/* ------------------------------------------------------------------ kv_cache ---- */

/* kv_paged_append / kv_paged_scatter: kernels/kv_cache/__init__.py:31-51,74-90;
 * semantics of torch_reference_kv_paged_append, triton_kv_paged.py:279-292:
 *   cache[slot / bs, :, slot % bs, :] = in[n]   for K and V.
 * Slots must be distinct. A slot outside [0, num_blocks*block_size) is skipped
 * (the reference's torch path wraps negatives Python-style and raises on overflow;
 * its .cu would write out of bounds, cuda_kv_paged.cu:33-38). */
typedef struct {
    const void* k_in;            /* [N, H_kv, D], strides below */
    const void* v_in;
    void* k_cache;               /* [num_blocks, H_kv, block_size, D] */
    void* v_cache;
    const int64_t* slot_mapping; /* [N] */
    int64_t n_tokens, num_kv_heads, head_dim, num_blocks, block_size;
    int64_t in_stride_n, in_stride_h;        /* shared by k_in and v_in; last dim contiguous */
    int64_t cache_stride_blk, cache_stride_h, cache_stride_pos; /* last dim contiguous */
    int dtype;                   /* rfx_dtype; a pure byte copy, any of the three */
    rfx_stream stream;
} RfxKvAppendArgs;
int rfx_kv_paged_append(const RfxKvAppendArgs* a);
int rfx_kv_paged_scatter(const RfxKvAppendArgs* a); /* same op, kv_cache/__init__.py:74-90 */

/* kv_paged_lookup: kernels/kv_cache/__init__.py:54-71; semantics of
 * torch_reference_kv_paged_lookup, triton_kv_paged.py:295-317:
 *   out[b, h, t, :] = cache[block_table[b, t / bs], h, t % bs, :]  for t < ctx_len[b],
 *   zero for t >= ctx_len[b] (K and V both; tests/test_kv_cache.py:117-122). */
typedef struct {
    const void* k_cache;
    const void* v_cache;
    void* k_out;                 /* [B, H_kv, max_ctx, D] contiguous, fully written */
    void* v_out;
    const int64_t* block_table;  /* [B, max_blocks] */
    const int32_t* context_lens; /* [B] */
    int64_t batch, num_kv_heads, head_dim, num_blocks, block_size, max_ctx, max_blocks;
    int64_t cache_stride_blk, cache_stride_h, cache_stride_pos;
    int64_t bt_stride_b;         /* block_table row stride, entries contiguous in a row */
    int dtype;
    rfx_stream stream;
} RfxKvLookupArgs;
int rfx_kv_paged_lookup(const RfxKvLookupArgs* a);

/* --------------------------------------------------------------------- rope ---- */

/* apply_rope / apply_rope_: kernels/rope/__init__.py:19-65; arithmetic of
 * torch_reference_rope, triton_rope.py:199-244: every multiply, subtract and add is
 * rounded to the activation dtype (the torch eager sequence), so 16-bit results are
 * bit-identical to the reference's torch path when the tables have the activation
 * dtype. Row s of cos/sin belongs to sequence index s. y may alias x (in place). */
typedef struct {
    const void* x;               /* logical [B, S, H, D]; strides below */
    void* y;
    const void* cos;             /* [S, D] in the activation dtype */
    const void* sin;
    int64_t batch, seq, heads, head_dim;
    int64_t x_stride_b, x_stride_s, x_stride_h;   /* last dim contiguous */
    int64_t y_stride_b, y_stride_s, y_stride_h;
    int64_t table_stride_s;
    int interleaved;             /* 0: pairs (i, i+D/2); 1: pairs (2i, 2i+1) */
    int dtype;
    rfx_stream stream;
} RfxRopeArgs;
int rfx_rope_apply(const RfxRopeArgs* a);

/* build_rope_tables: kernels/rope/triton_rope.py:247-285, computed on the device:
 * angle = pos*theta_i as one fp32 multiply (:269), cos/sin evaluated in fp64 of that
 * fp32 angle and rounded to fp32 (:270-271), duplicated to width D (:273-280), cast to
 * `dtype` (:285). theta_i = 1/base^(i/half) (:267) is read from inv_freq when given (so
 * a caller can pass the exact fp32 vector its own framework computes), else computed
 * here as 1.0f / (float)pow(base, (float)i/half). */
typedef struct {
    void* cos;                   /* [seq_len, D] contiguous */
    void* sin;
    const float* inv_freq;       /* [D/2] or NULL */
    int64_t seq_len, head_dim;
    double base;
    int interleaved;
    int dtype;
    rfx_stream stream;
} RfxRopeTableArgs;
int rfx_rope_build_tables(const RfxRopeTableArgs* a);

/* Fused RoPE + append (no single reference function; it is the composition
 * apply_rope(k_new) -> kv_paged_append of kernels/rope/__init__.py:19-39 and
 * kernels/kv_cache/__init__.py:31-51). Token n is rotated with table row positions[n];
 * K is rotated and written to the pool, V is copied; if q/q_out are given, Q is
 * rotated too (q_out may alias q). Cache contents equal the reference composition
 * bit for bit. */
typedef struct {
    const void* k_in;            /* [N, H_kv, D] contiguous */
    const void* v_in;
    const void* q_in;            /* [N, H_q, D] contiguous, or NULL */
    void* q_out;                 /* or NULL */
    void* k_cache;
    void* v_cache;
    const int64_t* slot_mapping; /* [N] */
    const int32_t* positions;    /* [N] row of the tables for token n */
    const void* cos;             /* [table_rows, D] activation dtype */
    const void* sin;
    int64_t n_tokens, num_q_heads, num_kv_heads, head_dim, num_blocks, block_size, table_rows;
    int64_t cache_stride_blk, cache_stride_h, cache_stride_pos;
    int interleaved;
    int dtype;
    rfx_stream stream;
    /* int8 pool (see the layout note at the top): k_cache/v_cache are int8, contiguous (the strides
     * above are ignored), and the rotated K rows and the V rows are quantised on the way in; their
     * scales go to k_scales/v_scales [num_blocks, num_kv_heads, block_size]. q_out stays in `dtype`. */
    int kv_int8;
    float* k_scales;
    float* v_scales;
} RfxRopeAppendArgs;
int rfx_rope_append(const RfxRopeAppendArgs* a);

/* ------------------------------------------------------------------ softmax ---- */

/* online_softmax: kernels/softmax/__init__.py:15-35; torch_reference_softmax,
 * triton_softmax.py:178-202. Rows of a [rows, n] contiguous matrix; causal masks
 * col > row % n (square contract, triton_softmax.py:66-69,146-164). Statistics in fp32. For
 * bf16 / fp16 rows the exponentials are rounded to the row's type once before they are scaled by
 * 1/sum (the sum is taken from the unrounded values), so a result can differ from the correctly
 * rounded one by one unit of the 16-bit type -- inside the reference's tolerances (bf16 2e-2,
 * fp16 1e-3, kernels/_common/dtype.py:47-52). x == y (in place) is allowed. */
typedef struct {
    const void* x;
    void* y;
    int64_t rows, n;
    int is_causal;
    int log;
    int dtype;
    rfx_stream stream;
} RfxSoftmaxArgs;
int rfx_online_softmax(const RfxSoftmaxArgs* a);

/* ---------------------------------------------------------------- attention ---- */

/* fused_attention (dense): kernels/attention/__init__.py:86-123; semantics of
 * torch_reference_attention, triton_fused_attention.py:350-371, with in-kernel GQA
 * h_kv = h / (H/H_kv) (triton_fused_attention.py:130-132), top-left causal
 * (:185-187), optional additive mask [B,H,S_q,S_k] (:190-202,303-308). */
typedef struct {
    const void* q;               /* [B, H, S_q, D] contiguous */
    const void* k;               /* [B, H_kv, S_k, D] contiguous */
    const void* v;
    void* out;                   /* [B, H, S_q, D] */
    const void* attn_mask;       /* same dtype as q, contiguous, or NULL */
    int64_t batch, num_q_heads, num_kv_heads, seq_q, seq_k, head_dim;
    float sm_scale;
    int is_causal;
    int dtype;
    void* workspace;             /* may be NULL when rfx_fused_attention_workspace_bytes() is 0 */
    size_t workspace_bytes;
    rfx_stream stream;
} RfxAttentionArgs;
size_t rfx_fused_attention_workspace_bytes(const RfxAttentionArgs* a);
int rfx_fused_attention(const RfxAttentionArgs* a);
/* Which kernel the arguments select: 1 = tcgen05 kernel (16-bit, head_dim 128, at least 32 query
 * rows per kv head, causal only with seq_q == seq_k, additive mask allowed, 16-byte aligned
 * tensors), 0 = scalar kernel, negative = invalid arguments. */
int rfx_fused_attention_kernel_kind(const RfxAttentionArgs* a);

/* Paged attention over ragged query chunks: the fused form of the composition
 * kv_paged_lookup -> repeat_interleave -> fused_attention evaluated per request with
 * max_ctx = context_lens[b] (kernels/kv_cache/__init__.py:54-71,
 * kernels/attention/__init__.py:86-123). Request b owns query rows
 * [q_start[b], q_start[b+1]) (one row per request when q_start is NULL: decode) and
 * keys 0..context_lens[b]-1, the new tokens included. Causal is bottom-right aligned:
 * query row i of n_b sees keys 0..context_lens[b]-n_b+i, the rule of
 * src/kernels/attention.cu:187. A request with no keys gives zeros
 * (src/kernels/attention.cu:163).
 *
 * Split-K: the work is cut into (request, kv_head, key-range) items by
 * rfx_paged_attention_plan, each item leaves an un-normalised (m, l, acc) partial in
 * the workspace, and rfx_splitk_combine merges them with the recurrence of
 * kernels/softmax/triton_softmax.py:84-89 / triton_fused_attention.py:205-227.
 * rfx_paged_attention runs plan (unless reuse_plan), partial kernel and combine; where the decode
 * kernel runs, the merge happens inside it (see rfx_paged_attention_partials_final) and the step is
 * two launches. */
typedef struct {
    const void* q;               /* [N_q, H_q, D] contiguous */
    void* out;                   /* [N_q, H_q, D] */
    const void* k_cache;         /* [num_blocks, H_kv, block_size, D] contiguous */
    const void* v_cache;
    const int64_t* block_table;  /* [B, max_blocks] */
    const int32_t* context_lens; /* [B] keys per request, new tokens included */
    const int32_t* q_start;      /* [B+1] or NULL (decode: row b belongs to request b) */
    /* optional RoPE fused into the Q load (rows rope_positions[n] of the tables) */
    const void* rope_cos;        /* [table_rows, D] activation dtype, or NULL */
    const void* rope_sin;
    const int32_t* rope_positions; /* [N_q] */
    int64_t n_q, batch, num_q_heads, num_kv_heads, head_dim;
    int64_t num_blocks, block_size, max_blocks, bt_stride_b, table_rows;
    int64_t max_q_len;           /* host upper bound of any request's query rows (1 for decode); sizes the
                                  * workspace and the grid. The device checks q_start against it and
                                  * against n_q: on a mismatch nothing is computed and status bit 2 is set */
    float sm_scale;
    int is_causal;               /* bottom-right; irrelevant when every request has one row */
    int rope_interleaved;
    int dtype;
    int reuse_plan;              /* 1: workspace already holds a plan for these lengths */
    int force_generic;           /* 1: use the scalar kernel (debug / parity cross-check) */
    int64_t target_chunk;        /* 0 = choose; >0 keys per split (rounded to 64); <0 query chunks are not split */
    void* workspace;
    size_t workspace_bytes;
    rfx_stream stream;
    /* int8 pool (see the layout note at the top): k_cache/v_cache are int8 and every key's score is
     * multiplied by its k scale, every probability by its v scale (the dequantisation of
     * src/kernels/attention.cu:91-96,141-150 moved behind the dot products; same value up to fp32
     * rounding). q, out and the RoPE tables stay in `dtype`. */
    int kv_int8;
    const float* k_scales;       /* [num_blocks, H_kv, block_size] */
    const float* v_scales;
} RfxPagedAttentionArgs;
size_t rfx_paged_attention_workspace_bytes(const RfxPagedAttentionArgs* a);
int rfx_paged_attention_plan(const RfxPagedAttentionArgs* a);
int rfx_paged_attention(const RfxPagedAttentionArgs* a);
/* The last two stages on their own, for callers that build their own launch sequence (a
 * CUDA graph, per-kernel timing): the split-K partial kernel over an existing plan, and
 * the combine that turns the partials into `out` and re-arms the plan for the next use. */
int rfx_paged_attention_partials(const RfxPagedAttentionArgs* a);
/* The decode kernel (kernel kind 1) can finish its rows itself: an item that is a whole (request, kv
 * head) pair writes `out` directly, and of a pair cut into several items the last one to finish merges
 * all their partials (a counter per pair in the workspace). rfx_paged_attention does exactly that and
 * launches no combine kernel then. This entry is that partial kernel alone, over an existing plan, for
 * callers that time or sequence the stages themselves; RFX_NOT_IMPLEMENTED for the other kernel kinds
 * (use rfx_paged_attention_partials + rfx_paged_attention_combine). */
int rfx_paged_attention_partials_final(const RfxPagedAttentionArgs* a);
/* Which kernel the arguments select: 2 = tcgen05 prefill kernel (16-bit, head_dim 128, ragged
 * query chunks given by q_start, queries already rotated, page size >= 8 dividing or a
 * multiple of 128; whole rows per CTA, or split over the keys with plan and combine when
 * max_q_len <= 512 and pages hold <= 64 keys), 3 = the same split batch with the decode
 * kernel launched in front of it for the requests of one query row (whenever the shapes fit that
 * kernel; it returns at once if the batch has none), 1 = TMA + warp-MMA decode kernel (16-bit, head_dim 64/128,
 * one query row per request, group <= 16, page size a divisor or multiple of 64 and >= 8),
 * 0 = scalar kernel, negative = invalid arguments. With kv_int8: 1 = the decode kernel's int8
 * instantiation (head_dim 128, one query row per request; K and V widened to fp16 in registers,
 * fp16 warp MMAs), 0 = scalar kernel for everything else. */
int rfx_paged_attention_kernel_kind(const RfxPagedAttentionArgs* a);
int rfx_paged_attention_combine(const RfxPagedAttentionArgs* a);

/* Paged attention for callers that cannot hand over a workspace. This entry point has no
 * counterpart in the reference. Some hosts of this library may not allocate device memory
 * at the point where they run attention: a runtime that took all of its memory up front and
 * forbids allocation afterwards, a plugin called inside someone else's memory pool, code on
 * a real-time path where cudaMalloc's implicit synchronisation is not acceptable. For them
 * the split-K plan and partials live in an 8 MiB array that is part of the library image
 * (rfx_paged_attention_static_capacity() bytes; every GPU that loads the library holds it
 * until the process exits). `workspace`, `workspace_bytes` and `reuse_plan` are ignored;
 * everything else is as for rfx_paged_attention, and so is the result. Problems whose
 * rfx_paged_attention_workspace_bytes() exceeds the capacity are rejected with
 * RFX_WORKSPACE_TOO_SMALL (an 8 MiB array covers e.g. 32 requests with 16 query / 2 kv heads
 * of head_dim 128, one query row each). The call allocates and frees nothing.
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current; the driver may load the array into
 * device memory at that moment); make that first call outside any stream capture. All calls on a device share the one array: it still holds the previous call's
 * plan and partials when the next call starts (each call rewrites what it reads, the status
 * word included), and two calls that overlap on the GPU -- different streams, or different
 * host threads -- race on it. Serialise them, or give the others a workspace of their own. */
size_t rfx_paged_attention_static_capacity(void);
int rfx_paged_attention_static(const RfxPagedAttentionArgs* a);

/* Split-K combine on caller-provided partials (the recurrence of
 * kernels/softmax/triton_softmax.py:84-89 with an accumulator,
 * triton_fused_attention.py:205-227): rows r = 0..rows-1 each own splits
 * [split_begin[r], split_begin[r+1]); out[r,:] = sum_s acc[s,:]*exp(m[s]-M) / sum_s l[s]*exp(m[s]-M). */
typedef struct {
    const float* acc;            /* [n_partials, D] */
    const float* m;              /* [n_partials] row maxima (natural-log domain) */
    const float* l;              /* [n_partials] */
    const int32_t* split_begin;  /* [rows+1] */
    void* out;                   /* [rows, D] in dtype */
    int64_t rows, head_dim;
    int dtype;
    rfx_stream stream;
} RfxCombineArgs;
int rfx_splitk_combine(const RfxCombineArgs* a);

/* Reads the device status word a paged-attention launch leaves in its workspace
 * (0 = ok; bit 0 = a bounded wait expired; bit 1 = a page index outside the pool: its keys
 * were left out; bit 2 = q_start disagrees with max_q_len or n_q: nothing was computed).
 * `workspace` NULL reads the word of rfx_paged_attention_static's built-in array on the
 * current device. Synchronises the stream; poll it after a step whose inputs are not trusted. */
int rfx_paged_attention_status(const void* workspace, rfx_stream stream, int* status_word_host);

/* ---- head-sharded output gather fused into the combine (no counterpart in the reference,
 * which has no multi-GPU code; the stock form of this step is an NCCL all-gather) ----------
 * Rank r of `world` ranks computes query heads [r*Hq, (r+1)*Hq) of every row, Hq =
 * num_q_heads of its RfxPagedAttentionArgs. With RfxHeadGatherArgs the combine kernel stores
 * each finished row slice straight into every rank's full output [n_q, world*Hq, D] through
 * peer-mapped pointers (plain stores over NVLink; nothing is read from a peer), then the last
 * CTA publishes `epoch` in every rank's flag array and, if `wait` is set, spins -- with an
 * iteration limit -- until every rank's flag on this GPU has reached `epoch`. When the kernel
 * has completed, peer_out[rank] holds all heads. `a->out` is not written.
 *
 * The caller owns every buffer. Because a peer may begin step k+1 while this rank still reads
 * the output of step k, alternate between two output buffers (epoch parity); the flags need
 * no reset: epochs only grow. On expiry of the wait bit 0 of the workspace status word is set
 * (rfx_paged_attention_status) and the kernel returns; the context stays usable.
 *
 * rfx_peer_export / rfx_peer_open / rfx_peer_close wrap the CUDA IPC calls that make a
 * cudaMalloc'ed buffer of another process addressable here (one process per GPU). */
#define RFX_MAX_PEERS 16
typedef struct {
    int world, rank;
    void* peer_out[RFX_MAX_PEERS];       /* [n_q, world*Hq, D] on each rank, as mapped in this process */
    uint32_t* peer_flags[RFX_MAX_PEERS]; /* [world] uint32 on each rank; slot [rank] is written by this rank */
    uint32_t* arrival_counter;           /* local device word, zero before the first use */
    uint32_t epoch;                      /* > 0, strictly increasing from step to step */
    int wait;                            /* 1: do not complete before every rank has published epoch */
    int64_t spin_limit;                  /* polls (about 100 ns each) before giving up; 0 = 10 million */
    /* Replayable form, for a step captured once in a CUDA graph (launch arguments are frozen at capture):
     * with epoch_word set, `epoch` is ignored; the kernel takes the step's epoch from that local device word
     * (its value + 1, the same for every CTA of the launch; the last CTA stores it back), and writes to
     * peer_out[p] + (epoch & 1) * out_alt_offset bytes, so peer_out[] then names the first of the two output
     * buffers of every rank. The word starts at zero and must not be written by anyone else. */
    uint32_t* epoch_word;
    int64_t out_alt_offset;
} RfxHeadGatherArgs;
/* Combine stage of rfx_paged_attention (after rfx_paged_attention_partials) with the gather. */
int rfx_paged_attention_combine_gather(const RfxPagedAttentionArgs* a, const RfxHeadGatherArgs* g);
/* All stages of rfx_paged_attention with the gathering combine. */
int rfx_paged_attention_gather(const RfxPagedAttentionArgs* a, const RfxHeadGatherArgs* g);

typedef struct {
    unsigned char handle[64]; /* cudaIpcMemHandle_t of the allocation that holds the pointer */
    int64_t offset;           /* of the pointer inside that allocation, bytes */
} RfxPeerHandle;
int rfx_peer_export(const void* device_ptr, RfxPeerHandle* out);
/* `mapped` = the exporting process's pointer as addressable here; `mapped_base` is what
 * rfx_peer_close takes. Must be called by a process other than the exporter. */
int rfx_peer_open(const RfxPeerHandle* h, void** mapped, void** mapped_base);
int rfx_peer_close(void* mapped_base);

/* ---- fused linear + norm (kernels/fused_linear_norm/__init__.py:27-73;
 * torch_reference_fused_linear_norm, kernels/fused_linear_norm/triton_kernel.py:204-233) ------
 *   y   = x @ weight^T + bias                       rounded to `dtype` (F.linear)
 *   out = layer_norm(y) * gamma + beta              (norm_type 0; one rounding at the end)
 *   out = round(y * rsqrt(mean(y^2) + eps)) * gamma (norm_type 1, RMSNorm; the product with gamma
 *                                                    is a second rounding in `dtype`, as in the reference)
 * x [M, K], weight [N, K], bias/gamma/beta [N] or NULL, out [M, N], all row-major and contiguous.
 * 16-bit dtypes with K % 8 == 0 and N % 8 == 0 run a tcgen05 GEMM (128x256 tiles, TMA-fed, fp32
 * accumulators in tensor memory) whose epilogue also leaves the row sums for the norm; the norm
 * is applied by a second, bandwidth-bound kernel over `out` in place. Up to 8 rows (decode) stream
 * the weights once with one warp per output column. Other cases (fp32, odd sizes) run a plain
 * shared-memory GEMM. The workspace holds the row statistics:
 * rfx_fused_linear_norm_workspace_bytes(args) bytes, 256-byte aligned. */
typedef struct {
    const void* x;
    const void* weight;
    const void* bias;            /* optional */
    const void* gamma;           /* optional */
    const void* beta;            /* optional, layer norm only */
    void* out;
    int64_t M, K, N;
    float eps;
    int norm_type;               /* 0 = LayerNorm, 1 = RMSNorm */
    int dtype;
    int force_generic;           /* 1 = the plain GEMM even where the tcgen05 one applies (testing) */
    void* workspace;
    size_t workspace_bytes;
    rfx_stream stream;
} RfxLinearNormArgs;
size_t rfx_fused_linear_norm_workspace_bytes(const RfxLinearNormArgs* a);
int rfx_fused_linear_norm(const RfxLinearNormArgs* a);
/* 1 = tcgen05 GEMM, 2 = weight-streaming kernel for up to 8 rows (16-bit), 0 = plain GEMM,
 * negative = invalid arguments. */
int rfx_fused_linear_norm_kernel_kind(const RfxLinearNormArgs* a);

#ifdef __cplusplus
}
#endif
#endif /* REFLEX_B200_H_ */
