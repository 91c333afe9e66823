// Paged GQA decode, split-K partial kernel for 16-bit KV with head_dim 128 or 64.
//
// HBM-bound: every item (a run of 64-key tiles of one (request, kv_head) pair) streams its
// K and V pages exactly once. One persistent CTA per SM owns one equal run of the tile
// stream; it has four producer warps and one or two groups of four consumer warps:
//   producers: each loads the run's item descriptors in one round trip, keeps the block-table
//              entries of the current and the next item in registers (32 per lane-window), and
//              fills the stages whose number in the CTA's sequence is its own modulo four: one
//              TMA tile copy per page for K and for V into a ring of 64-key stages; each copy
//              lands the page as [half][row][128 B] with the 128-byte swizzle, completion counted
//              on the stage's mbarrier. With an item's first stage go the G query rows and the
//              RoPE table rows. (Filling a stage costs a warp 1200-1900 cycles -- a barrier
//              poll, the page look-up, 90 cycles per copy instruction -- while the stage's bytes
//              arrive in 770-1500: a single producer warp was the limit of the kernel.)
//   consumers: each warp takes 16 of the stage's 64 keys as the 16 MMA rows and the group's
//              heads as the columns: S^T = K.Q^T, softmax down the columns, O^T += V^T.P^T,
//              all through m16n8k16 warp MMAs fed by conflict-free ldmatrix. At the item's
//              last stage the warps merge (m, l, acc) through shared memory. With two groups,
//              stages alternate between them (a lone warp per scheduler runs at a third of an
//              instruction per cycle; two hide each other's latencies).
// An item that is a whole pair writes its output rows directly; of a pair cut into several
// items the last one to finish merges the partials of all (a counter per pair), so that no
// combine kernel follows. RoPE is fused into the Q load with torch's per-op rounding.
// int8 pools (one fp32 scale per position and kv head) widen K and V to fp16 in registers
// and run the same MMAs in fp16; the scales multiply the scores and the probabilities.
//
// Algorithmic bytes per item: 2 * keys * D * e (K and V). Arithmetic is G FLOP/byte, far
// below what the warp MMA path sustains; the kernel's roofline is HBM bandwidth.
#include <stdlib.h>

#include <mutex>
#include <type_traits>

#include "paged_plan.cuh"
#include "ptx.cuh"

namespace rfx {

constexpr int kTile = kPlanTile;    // keys per stage
constexpr int kGroupWarps = 4;      // warps per consumer group, 16 keys each
constexpr int kProducers = 4;       // producer warps; stage n of a CTA's sequence belongs to warp n % 4
constexpr int kAccPad = 4;          // floats of padding per merge row (bank spread)

struct alignas(16) StageMeta {  // 32 bytes: the mbarriers behind the array stay 8-byte aligned
    int item;      // -1: no more work
    int n_valid;   // keys of this stage that exist (0..64)
    int flags;     // bit0 first stage of item, bit1 last stage of item, bit2 rotate Q
    int prow;      // first partial row of the item
    unsigned bad;  // boxes of the stage that were not loaded (page index outside the pool): their keys do not count
    int pair;      // request * Hkv + kv head
    int item0;     // first item of the pair
    int ns;        // items of the pair (1: the item is the whole pair)
};

struct DecodeParams {
    const void* q;
    const int32_t* q_start;  // mixed batches: the kernel takes the requests with one query row, at row q_start[b]
    const int64_t* block_table;
    const void* rcos;
    const void* rsin;
    const int32_t* rpos;
    int32_t* hdr;
    const int32_t* part_first;
    const int4* items;
    const int32_t* item_prow;
    float* pm;
    float* pl;
    float* pacc;
    int64_t num_blocks, max_blocks, bt_sb, table_rows;
    int Hq, Hkv, G, block_size, box_rows, rope_inter;
    int map2d;         // 1: the maps are 2-D [rows, D] with {64, box_rows} boxes, one copy per 128-byte half
    float scale_log2;  // sm_scale * log2(e)
    const float* k_scales;  // int8 pool: one fp32 scale per (page, kv head, position), else nullptr
    const float* v_scales;
    // Merge inside the kernel (out != nullptr): an item that is a whole pair writes its output rows
    // itself; of a pair cut into several items the last one to finish merges the partials of all. Then
    // no combine kernel follows. pair_counter[B*Hkv] counts the finished items of each pair (zero
    // between launches: the last arriver puts it back).
    void* out;
    const int32_t* pair_item_begin;
    int32_t* pair_counter;
    int n_pairs;
    int late_trigger;  // 1: dependents may start only once this kernel's own predecessors are done (see the kernel)
};

template <int HD, int GP, int STAGES, bool Q8 = false>
struct DecodeSmem {
    static constexpr int kRowBytes = HD * 2;              // a query or table row (16-bit)
    static constexpr int kKvRowBytes = Q8 ? HD : HD * 2;  // a key or value row
    static constexpr int kTileBytes = kTile * kKvRowBytes;  // K or V of one stage
    static constexpr int kAccStride = HD + kAccPad;
    static constexpr int kQBytes = GP * kRowBytes;        // raw query rows of the group
    static constexpr int kQSlot = kQBytes + 2 * kRowBytes;  // + cos row + sin row
    static constexpr int kScaleSlot = Q8 ? 2 * kTile * 4 : 0;  // int8: the stage's K scales, then its V scales
    static constexpr size_t off_k = 0;
    static constexpr size_t off_v = (size_t)STAGES * kTileBytes;
    static constexpr size_t off_sc = 2 * (size_t)STAGES * kTileBytes;
    static constexpr size_t off_q = off_sc + (size_t)STAGES * kScaleSlot;
    static constexpr size_t off_merge = off_q + (size_t)STAGES * kQSlot;
    static constexpr size_t merge_bytes = (size_t)kGroupWarps * GP * kAccStride * 4;
    static constexpr size_t off_ml = off_merge + merge_bytes;             // [group warps][GP][2]
    static constexpr size_t off_meta = off_ml + (size_t)kGroupWarps * GP * 2 * 4 + 16;  // + the "last item of its pair" flag
    static constexpr size_t off_bars = off_meta + (size_t)STAGES * sizeof(StageMeta);
    static_assert(sizeof(StageMeta) % 8 == 0 && off_meta % 8 == 0, "mbarriers need 8-byte alignment");
    static constexpr size_t total = off_bars + 2 * (size_t)STAGES * 8 + 1024;  // + alignment slack
};

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
    __device__ static uint32_t pack(float a, float b) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
};
template <> struct Pack2<__half> {
    __device__ static uint32_t pack(float a, float b) {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
};

template <typename T> __device__ inline uint32_t pack_t(T a, T b) {
    const uint16_t lo = *reinterpret_cast<uint16_t*>(&a), hi = *reinterpret_cast<uint16_t*>(&b);
    return (uint32_t)lo | ((uint32_t)hi << 16);
}

// Four int8 (two's complement) in `wx`, already xor-ed with 0x80 (value + 128 as an unsigned byte): the two
// picked by `sel` (a byte-permute selector that puts each next to the byte 0x64) become fp16 1024 + byte;
// minus 1152 gives the signed value, exactly.
__device__ __forceinline__ uint32_t q8_pair_to_h2(uint32_t wx, uint32_t sel) {
    uint32_t t = __byte_perm(wx, 0x64646464u, sel);
    const uint32_t bias = 0x64806480u;  // 1152.0, twice
    __half2 r = __hsub2(*reinterpret_cast<__half2*>(&t), *reinterpret_cast<const __half2*>(&bias));
    return *reinterpret_cast<uint32_t*>(&r);
}

// The same without the subtraction: fp16 value + 1152. The decode kernel feeds K like this to the MMAs and
// takes the offset out of the scores (1152 times the sum of the head's query values), which saves the two
// packed subtractions per 32-bit word of K: a score sums 128 products, so the offset costs no accuracy
// worth the name. V keeps the exact form: its products are summed over the whole context, and with the
// offset carried along the output error was measured at 7.6e-4 instead of 1.2e-4 (8-32 k keys).
__device__ __forceinline__ uint32_t q8_pair_biased(uint32_t wx, uint32_t sel) { return __byte_perm(wx, 0x64646464u, sel); }
constexpr float kQ8Bias = 1152.f;

// Two elements of T side by side in the type the warp MMA runs in: T itself, or fp16 when the pool is
// int8 (the widened K and V are fp16, so Q has to be too; a bf16 value is exact in fp16 unless it is
// below 2^-14 in magnitude or above 65504).
template <typename T, bool Q8> __device__ inline uint32_t pack_mma(T a, T b) {
    if (Q8 && !std::is_same<T, __half>::value) {
        __half2 h = __floats2half2_rn(Num<T>::to_f(a), Num<T>::to_f(b));
        return *reinterpret_cast<uint32_t*>(&h);
    }
    const uint16_t lo = *reinterpret_cast<uint16_t*>(&a), hi = *reinterpret_cast<uint16_t*>(&b);
    return (uint32_t)lo | ((uint32_t)hi << 16);
}

// Builds the A fragments of Q for the item's G heads from the stage's query slot
// (raw rows, then the cos row, then the sin row), rotating when asked.
// qa[ks][0] = row g,   dims 16ks + 2c + {0,1};   qa[ks][1] = row g+8, same dims;
// qa[ks][2] = row g,   dims 16ks + 8 + 2c + ..;  qa[ks][3] = row g+8      (c = lane % 4).
//
// Q8 (int8 pool): ldmatrix hands a thread four consecutive int8 of a key row, i.e. dims 4c..4c+3 of a
// 16-dim chunk, so the contraction index of the MMA is permuted inside each chunk: MMA columns
// 2c, 2c+1 stand for dims 4c, 4c+1 and columns 2c+8, 2c+9 for dims 4c+2, 4c+3. The Q fragments follow.
template <typename T, int HD, int GP, bool Q8>
__device__ inline void load_q_frags(uint32_t (&qa)[HD / 16][4], const unsigned char* slot, int G, bool rotate,
                                    bool interleaved, float (&qsum)[GP / 8]) {
    const int lane = threadIdx.x & 31;
    const int g0 = lane >> 2, c = lane & 3;
    const T* qs = reinterpret_cast<const T*>(slot);
    const T* cr = qs + GP * HD;
    const T* sr = cr + HD;
    if constexpr (Q8) {
#pragma unroll
        for (int rr = 0; rr < (GP > 8 ? 2 : 1); ++rr) {
            const int g = g0 + 8 * rr;
            const bool live = g < G;
            const T* qr = qs + g * HD;
            float acc = 0.f;  // sum of this head's query values as the MMA sees them (fp16)
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                T y[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int d = 16 * ks + 4 * c + e;
                    y[e] = live ? qr[d] : Num<T>::from_f(0.f);
                    if (live && rotate) {
                        T y1, y2;
                        if (interleaved) {
                            const int d0 = d & ~1;
                            rope_pair<T>(qr[d0], qr[d0 + 1], cr[d0], sr[d0], y1, y2);
                            y[e] = (d & 1) ? y2 : y1;
                        } else {
                            const int d0 = d < HD / 2 ? d : d - HD / 2;
                            rope_pair<T>(qr[d0], qr[d0 + HD / 2], cr[d0], sr[d0], y1, y2);
                            y[e] = d < HD / 2 ? y1 : y2;
                        }
                    }
                }
                qa[ks][rr] = pack_mma<T, true>(y[0], y[1]);
                qa[ks][2 + rr] = pack_mma<T, true>(y[2], y[3]);
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][rr]));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][2 + rr]));
                acc += (f0.x + f0.y) + (f1.x + f1.y);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            qsum[rr] = acc;  // the same in the four lanes that share the head
        }
        if (GP <= 8) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) { qa[ks][1] = 0; qa[ks][3] = 0; }
        }
    } else {
#pragma unroll
    for (int rr = 0; rr < (GP > 8 ? 2 : 1); ++rr) {
        const int g = g0 + 8 * rr;
        const bool live = g < G;
        const T* qr = qs + g * HD;
        if (!rotate) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                uint32_t lo = 0, hi = 0;
                if (live) {
                    lo = *reinterpret_cast<const uint32_t*>(qr + 16 * ks + 2 * c);
                    hi = *reinterpret_cast<const uint32_t*>(qr + 16 * ks + 8 + 2 * c);
                }
                qa[ks][rr] = lo;
                qa[ks][2 + rr] = hi;
            }
        } else if (interleaved) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int d = 16 * ks + 8 * hh + 2 * c;
                    uint32_t r = 0;
                    if (live) {
                        T y1, y2;
                        rope_pair<T>(qr[d], qr[d + 1], cr[d], sr[d], y1, y2);
                        r = pack_t<T>(y1, y2);
                    }
                    qa[ks][2 * hh + rr] = r;
                }
            }
        } else {
            // pairs (d, d + HD/2): k-steps ks and ks + HD/32 hold the partners
#pragma unroll
            for (int ks = 0; ks < HD / 32; ++ks) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int d = 16 * ks + 8 * hh + 2 * c;
                    uint32_t r1 = 0, r2 = 0;
                    if (live) {
                        T a1, a2, b1, b2;
                        rope_pair<T>(qr[d], qr[d + HD / 2], cr[d], sr[d], a1, a2);
                        rope_pair<T>(qr[d + 1], qr[d + 1 + HD / 2], cr[d + 1], sr[d + 1], b1, b2);
                        r1 = pack_t<T>(a1, b1);
                        r2 = pack_t<T>(a2, b2);
                    }
                    qa[ks][2 * hh + rr] = r1;
                    qa[ks + HD / 32][2 * hh + rr] = r2;
                }
            }
        }
    }
    if (GP <= 8) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) { qa[ks][1] = 0; qa[ks][3] = 0; }
    }
}  // not Q8
}

template <typename T, int HD, int GP, int STAGES, int GROUPS, bool Q8>
__global__ void __launch_bounds__((kGroupWarps * GROUPS + kProducers) * 32, 1)
decode_mma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  const DecodeParams P) {
    using S = DecodeSmem<HD, GP, STAGES, Q8>;
    constexpr bool BF = std::is_same<T, __nv_bfloat16>::value && !Q8;  // the type of the warp MMAs
    using PT = typename std::conditional<Q8, __half, T>::type;         // ... and of the packed probabilities
    constexpr int kConsumers = kGroupWarps * GROUPS;
    extern __shared__ unsigned char smem_raw[];
    // TMA's 128-byte swizzle is a function of the shared-memory address, so tiles must
    // start on 1024-byte boundaries; the launch asks for 1 KiB of slack.
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* sK = smem + S::off_k;
    unsigned char* sV = smem + S::off_v;
    unsigned char* sQ = smem + S::off_q;
    float* sScale = reinterpret_cast<float*>(smem + S::off_sc);  // int8 pool only
    float* sAcc = reinterpret_cast<float*>(smem + S::off_merge);
    float* sML = reinterpret_cast<float*>(smem + S::off_ml);
    StageMeta* sMeta = reinterpret_cast<StageMeta*>(smem + S::off_meta);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::off_bars);
    uint64_t* empty = full + STAGES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = P.box_rows;                 // rows per TMA box = min(block_size, 64)
    const uint32_t box_bytes = (uint32_t)R * S::kKvRowBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], kConsumers);
        }
        ptx::fence_barrier_init();
    }
    __syncthreads();
    // The kernel behind this one may be scheduled already: the combine kernel waits for this one itself.
    // When this kernel takes the one-row requests of a mixed batch, the kernel behind it is the chunked
    // prefill kernel, which reads the same plan and does not wait for this kernel until its own end (its
    // CTAs fill the SMs this kernel's CTAs leave): it must not start before the plan is complete, so the
    // trigger comes after this kernel's own wait.
    if (!P.late_trigger) ptx::pdl_trigger();
    ptx::pdl_wait();     // everything below reads what earlier kernels wrote (plan, pool, Q)
    if (P.late_trigger) ptx::pdl_trigger();
    // a mixed batch without one-row requests: nothing here is this kernel's (uniform over the grid)
    if (P.q_start != nullptr && P.hdr[HdrOneRowRequests] == 0) return;

    if (warp >= kConsumers) {  // the last warps
        // ------------------------------------------------------------ producers --
        // Filling a stage costs its producer well over a thousand cycles (a barrier poll, the page
        // look-up, one instruction per copy, each a round trip to a unit that is busy), more than the
        // stage's bytes take to arrive, so four warps share the work: every one walks the whole run
        // (the bookkeeping is cheap) and fills the stages whose number in the CTA's sequence is its own
        // modulo four. A ring slot is therefore always filled by one warp at a time.
        const int pw = warp - kConsumers;
        if (lane == 0 && pw == 0) {
            ptx::prefetch_tensormap(&kmap);
            ptx::prefetch_tensormap(&vmap);
        }
        // The CTA's first run: its bounds are asked for together with the number of runs (the array has an
        // entry for every run the launch could have), one round trip instead of two before the first copy.
        int first_begin = P.part_first[blockIdx.x], first_end = P.part_first[blockIdx.x + 1];
        const int n_parts = P.hdr[HdrNumParts];
        int stage = 0;
        uint32_t phase = 0;
        int turn = 0;  // whose stage comes next
        bool alive = true;
        for (int part = blockIdx.x; part < n_parts && alive; part += gridDim.x) {
            const int i_begin = part == (int)blockIdx.x ? first_begin : P.part_first[part];
            const int i_end = part == (int)blockIdx.x ? first_end : P.part_first[part + 1];
            for (int ib = i_begin; ib < i_end && alive; ib += 32) {
                // one round trip: lane j holds the descriptor of item ib + j
                const int my_id = ib + lane;
                int4 my_desc = make_int4(0, 0, 0, 0);
                int my_prow = 0, my_pos = -1, my_qrow = -1, my_item0 = 0, my_ns = 1;
                if (my_id < i_end) {
                    my_desc = P.items[my_id];
                    my_prow = P.item_prow[my_id];
                    if (P.out) {
                        const int pr = my_desc.x * P.Hkv + my_desc.y;
                        my_item0 = P.pair_item_begin[pr];
                        my_ns = P.pair_item_begin[pr + 1] - my_item0;
                    }
                    if (P.rcos) my_pos = P.rpos[my_desc.x];
                    my_qrow = my_desc.x;
                    if (P.q_start) {
                        const int r0 = P.q_start[my_desc.x];
                        my_qrow = (P.q_start[my_desc.x + 1] - r0 == 1) ? r0 : -1;  // other requests: not this kernel's
                    }
                }
                const int n_here = min(32, i_end - ib);
                auto load_win = [&](const int64_t* bt, int w0, int ke) -> int64_t {
                    const int64_t lb = (int64_t)w0 + lane;
                    const int64_t last = ((int64_t)ke - 1) / P.block_size;
                    return (lb <= last && lb < P.max_blocks) ? bt[lb] : -1;
                };
                // block-table window of the first item; later items prefetch during their predecessor
                int64_t nx_cur, nx_nxt;
                {
                    const int b0 = __shfl_sync(0xffffffffu, my_desc.x, 0);
                    const int kb0 = __shfl_sync(0xffffffffu, my_desc.z, 0), ke0 = __shfl_sync(0xffffffffu, my_desc.w, 0);
                    const int64_t* bt0 = P.block_table + (int64_t)b0 * P.bt_sb;
                    nx_cur = load_win(bt0, kb0 / P.block_size, ke0);
                    nx_nxt = load_win(bt0, kb0 / P.block_size + 32, ke0);
                }
                for (int j = 0; j < n_here && alive; ++j) {
                    const int b = __shfl_sync(0xffffffffu, my_desc.x, j), hkv = __shfl_sync(0xffffffffu, my_desc.y, j);
                    const int kb = __shfl_sync(0xffffffffu, my_desc.z, j), ke = __shfl_sync(0xffffffffu, my_desc.w, j);
                    const int prow = __shfl_sync(0xffffffffu, my_prow, j);
                    const int pos = __shfl_sync(0xffffffffu, my_pos, j);
                    const int qrow = __shfl_sync(0xffffffffu, my_qrow, j);
                    const int item0 = __shfl_sync(0xffffffffu, my_item0, j), ns = __shfl_sync(0xffffffffu, my_ns, j);
                    const bool rotate = P.rcos != nullptr && pos >= 0 && (int64_t)pos < P.table_rows;
                    const int64_t* bt = P.block_table + (int64_t)b * P.bt_sb;
                    int win0 = kb / P.block_size;
                    int64_t pg_cur = nx_cur, pg_nxt = nx_nxt;
                    if (j + 1 < n_here) {
                        const int b1 = __shfl_sync(0xffffffffu, my_desc.x, j + 1);
                        const int kb1 = __shfl_sync(0xffffffffu, my_desc.z, j + 1);
                        const int ke1 = __shfl_sync(0xffffffffu, my_desc.w, j + 1);
                        const int64_t* bt1 = P.block_table + (int64_t)b1 * P.bt_sb;
                        nx_cur = load_win(bt1, kb1 / P.block_size, ke1);
                        nx_nxt = load_win(bt1, kb1 / P.block_size + 32, ke1);
                    }
                    if (qrow < 0) continue;
                    const int n_tiles = (ke - kb + kTile - 1) / kTile;
                    for (int t = 0; t < n_tiles && alive; ++t) {
                        const int tok0 = kb + t * kTile;
                        const bool mine = turn == pw;
                        if (++turn == kProducers) turn = 0;
                        if (!mine) {
                            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                            const int next_lb = (tok0 + kTile) / P.block_size;
                            if (next_lb - win0 >= 32 && t + 1 < n_tiles) {
                                win0 += 32;
                                pg_cur = pg_nxt;
                                pg_nxt = load_win(bt, win0 + 32, ke);
                            }
                            continue;
                        }
                        const int n_valid = min(kTile, ke - tok0);
                        const int n_boxes = (n_valid + R - 1) / R;
                        int ok = 1;
                        if (lane == 0) ok = ptx::mbar_wait_bounded(&empty[stage], phase ^ 1u) ? 1 : 0;
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if (!ok) {
                            if (lane == 0) atomicOr(P.hdr + HdrStatus, kStatusWaitExpired);
                            alive = false;
                            break;
                        }
                        // page of box i: logical block (tok0 + i*R) / block_size
                        int64_t my_page = -1;
                        int my_row0 = 0;
                        {
                            const bool want = lane < n_boxes;
                            const int tok = tok0 + (want ? lane : 0) * R;
                            const int lb = tok / P.block_size;
                            my_row0 = tok - lb * P.block_size;
                            const int rel = lb - win0;  // 0..63 by construction of the window advance
                            const int64_t a = __shfl_sync(0xffffffffu, pg_cur, rel & 31);
                            const int64_t c2 = __shfl_sync(0xffffffffu, pg_nxt, rel & 31);
                            if (want) my_page = rel < 32 ? a : c2;
                        }
                        const bool page_ok = my_page >= 0 && my_page < P.num_blocks;
                        const unsigned okmask = __ballot_sync(0xffffffffu, lane < n_boxes && page_ok);
                        const unsigned wantmask = __ballot_sync(0xffffffffu, lane < n_boxes);
                        const uint32_t q_bytes = (uint32_t)P.G * S::kRowBytes;
                        if (lane == 0) {
                            StageMeta m;
                            m.item = ib + j; m.n_valid = n_valid;
                            m.flags = (t == 0 ? 1 : 0) | (t == n_tiles - 1 ? 2 : 0) | (rotate ? 4 : 0);
                            m.prow = prow;
                            m.bad = wantmask & ~okmask;
                            m.pair = b * P.Hkv + hkv; m.item0 = item0; m.ns = ns;
                            sMeta[stage] = m;
                            if (okmask != wantmask) atomicOr(P.hdr + HdrStatus, kStatusBadPage);
                            uint32_t tx = (2u * box_bytes + (Q8 ? 8u * (uint32_t)R : 0u)) * (uint32_t)__popc(okmask);
                            if (t == 0) tx += q_bytes + (rotate ? 2u * S::kRowBytes : 0u);
                            ptx::mbar_arrive_expect_tx(&full[stage], tx);
                        }
                        __syncwarp();
                        if (lane < n_boxes && page_ok) {
                            const int row = (int)((my_page * P.Hkv + hkv) * P.block_size + my_row0);
                            unsigned char* kd = sK + (size_t)stage * S::kTileBytes + (size_t)lane * box_bytes;
                            unsigned char* vd = sV + (size_t)stage * S::kTileBytes + (size_t)lane * box_bytes;
                            if (Q8) {
                                // a row is one 128-byte line; the scales of the box's keys ride along
                                ptx::tma_load_2d(kd, &kmap, &full[stage], 0, row);
                                ptx::tma_load_2d(vd, &vmap, &full[stage], 0, row);
                                float* sc = sScale + (size_t)stage * (2 * kTile) + lane * R;
                                ptx::bulk_load(sc, P.k_scales + row, (uint32_t)R * 4u, &full[stage]);
                                ptx::bulk_load(sc + kTile, P.v_scales + row, (uint32_t)R * 4u, &full[stage]);
                            } else if (!P.map2d) {
                                ptx::tma_load_3d(kd, &kmap, &full[stage], 0, row, 0);
                                ptx::tma_load_3d(vd, &vmap, &full[stage], 0, row, 0);
                            } else {
#pragma unroll
                                for (int hf = 0; hf < HD / 64; ++hf) {
                                    ptx::tma_load_2d(kd + (size_t)hf * R * 128, &kmap, &full[stage], hf * 64, row);
                                    ptx::tma_load_2d(vd + (size_t)hf * R * 128, &vmap, &full[stage], hf * 64, row);
                                }
                            }
                        }
                        if (t == 0 && lane == 31) {
                            // the item's query rows (contiguous: heads hkv*G .. hkv*G+G-1 of row b) and table rows
                            unsigned char* qd = sQ + (size_t)stage * S::kQSlot;
                            const unsigned char* qsrc = (const unsigned char*)P.q +
                                                        ((int64_t)qrow * P.Hq + (int64_t)hkv * P.G) * S::kRowBytes;
                            ptx::bulk_load(qd, qsrc, q_bytes, &full[stage]);
                            if (rotate) {
                                ptx::bulk_load(qd + S::kQBytes, (const unsigned char*)P.rcos + (int64_t)pos * S::kRowBytes,
                                               S::kRowBytes, &full[stage]);
                                ptx::bulk_load(qd + S::kQBytes + S::kRowBytes,
                                               (const unsigned char*)P.rsin + (int64_t)pos * S::kRowBytes, S::kRowBytes,
                                               &full[stage]);
                            }
                        }
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                        // advance the block window once the next stage starts beyond it
                        const int next_lb = (tok0 + kTile) / P.block_size;
                        if (next_lb - win0 >= 32 && t + 1 < n_tiles) {
                            win0 += 32;
                            pg_cur = pg_nxt;
                            pg_nxt = load_win(bt, win0 + 32, ke);
                        }
                    }
                }
            }
        }
        // Tell the consumers there is nothing left (the warp whose turn it is).
        if (alive && lane == 0 && turn == pw) {
            if (ptx::mbar_wait_bounded(&empty[stage], phase ^ 1u)) {
                StageMeta m;
                m.item = -1; m.n_valid = 0; m.flags = 0; m.prow = 0; m.bad = 0; m.pair = 0; m.item0 = 0; m.ns = 1;
                sMeta[stage] = m;
                ptx::mbar_arrive(&full[stage]);
            } else {
                atomicOr(P.hdr + HdrStatus, kStatusWaitExpired);
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers --
    // Keys are the 16 MMA rows and the group's heads the columns: S^T = K.Q^T (A = K rows
    // straight from the swizzled tile, B = the Q fragments), softmax down the columns with
    // lane/4 shuffles, P^T turned into a B operand with movmatrix, O^T += V^T.P^T (A = V
    // through transposing ldmatrix). No MMA row or column is padding when G is 8 or 16.
    constexpr int NT = GP / 8;  // head n-tiles
    const int group = warp / kGroupWarps, wq = warp % kGroupWarps;
    const int r8 = lane >> 2, c4 = lane & 3;
    // dims (inside a 16-dim block) of the accumulator rows r8 and r8 + 8 of this thread
    const int dim_lo = Q8 ? 2 * r8 : r8, dim_hi = Q8 ? 2 * r8 + 1 : 8 + r8;
    uint32_t qa[HD / 16][4];
    float o[HD / 16][NT][4];
    float m_run[NT][2], l_run[NT][2];
    // int8 pool: K enters the MMAs with an offset of 1152 (see q8_pair_biased); qoff = 1152 x the sum of the
    // head's query values is taken out of the scores.
    [[maybe_unused]] float qoff[NT][2];

    // lane-constant parts of the ldmatrix addresses
    const int mat = lane >> 3, rowi = lane & 7;
    const int k_tok = wq * 16 + (mat & 1) * 8 + rowi;   // K (A operand): matrices 0,2 keys 0-7; 1,3 keys 8-15
    const int v_tok = wq * 16 + (mat >> 1) * 8 + rowi;  // V (A operand, transposed): matrices 0,1 keys 0-7; 2,3 keys 8-15
    const int k_box = k_tok / R, k_r = k_tok - k_box * R;
    const int v_box = v_tok / R, v_r = v_tok - v_box * R;
    const uint32_t k_rowoff = (uint32_t)k_box * box_bytes + (uint32_t)k_r * 128u;  // int8: a row is one 128-byte line
    const uint32_t v_rowoff = (uint32_t)v_box * box_bytes + (uint32_t)v_r * 128u;
    const uint32_t half_bytes = (uint32_t)R * 128u;
    const uint32_t k_sw = (uint32_t)(k_r & 7), v_sw = (uint32_t)(v_r & 7);
    const uint32_t sK_u32 = ptx::smem_u32(sK), sV_u32 = ptx::smem_u32(sV);

    if (P.out) {
        // A request without keys has no item: nobody else would write its output rows (zeros).
        T* outp = static_cast<T*>(P.out);
        for (int pr = blockIdx.x * kConsumers + warp; pr < P.n_pairs; pr += gridDim.x * kConsumers) {
            if (P.pair_item_begin[pr + 1] != P.pair_item_begin[pr]) continue;
            const int b = pr / P.Hkv, hkv = pr - b * P.Hkv;
            T* orow = outp + ((int64_t)b * P.Hq + (int64_t)hkv * P.G) * HD;
            for (int i = lane; i < P.G * HD; i += 32) orow[i] = Num<T>::from_f(0.f);
        }
    }
    int stage = 0;
    uint32_t phase = 0;
    int turn = 0;  // which group computes the current stage
    while (true) {
        // every lane acquires the stage itself; the vote keeps an expired wait warp-uniform
        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(&full[stage], phase) ? 1 : 0)) {
            if (lane == 0) atomicOr(P.hdr + HdrStatus, kStatusWaitExpired);
            break;
        }
        const StageMeta meta = sMeta[stage];
        if (meta.item < 0) break;
        if (meta.flags & 1) {
            float qsum[NT];
            load_q_frags<T, HD, GP, Q8>(qa, sQ + (size_t)stage * S::kQSlot, P.G, (meta.flags & 4) != 0, P.rope_inter != 0, qsum);
            if (Q8) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        qoff[nt][i] = kQ8Bias * __shfl_sync(0xffffffffu, qsum[nt], (2 * c4 + i) * 4);  // head 8 nt + 2 c4 + i
                    }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) { m_run[nt][0] = m_run[nt][1] = -INFINITY; l_run[nt][0] = l_run[nt][1] = 0.f; }
#pragma unroll
            for (int j = 0; j < HD / 16; ++j)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[j][nt][i] = 0.f;
        }
        const int slice0 = wq * 16;
        if (group == turn && slice0 < meta.n_valid) {
            const uint32_t kst = sK_u32 + (uint32_t)stage * S::kTileBytes;
            const uint32_t vst = sV_u32 + (uint32_t)stage * S::kTileBytes;
            // Keys past the end, and keys of a page whose index is outside the pool, do not count. What
            // sits in their rows may be anything (stale pages, NaN patterns): their probabilities are
            // zero but 0*NaN would poison P.V, so those V rows are cleared.
            const bool tail = meta.n_valid < slice0 + 16 || meta.bad != 0;
            auto dead = [&](int tk) -> bool { return tk >= meta.n_valid || ((meta.bad >> (tk / R)) & 1u); };
            if (tail && !Q8) {
                unsigned char* vs = sV + (size_t)stage * S::kTileBytes;
                for (int i = lane; i < 16 * (S::kRowBytes / 16); i += 32) {
                    const int tk = slice0 + i / (S::kRowBytes / 16);
                    const int ch = i % (S::kRowBytes / 16);
                    if (dead(tk)) {
                        const int bx = tk / R, rr = tk - bx * R;
                        *reinterpret_cast<uint4*>(vs + (size_t)bx * box_bytes + (size_t)(ch >> 3) * half_bytes +
                                                  (size_t)rr * 128 + (size_t)(ch & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
            }
            // ---- S^T = K.Q^T : rows = this warp's 16 keys, cols = heads of the group
            float s[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
            // int8 pool: the scales of this thread's two keys (rows r8 and r8 + 8 of the slice); a key that
            // does not count gets a zero V scale, since its scale word may be anything
            float ksl[2] = {P.scale_log2, P.scale_log2}, vsc[2] = {1.f, 1.f};
            if (Q8) {
                const float* sc = sScale + (size_t)stage * (2 * kTile) + slice0 + r8;
                ksl[0] = sc[0] * P.scale_log2; ksl[1] = sc[8] * P.scale_log2;
                vsc[0] = sc[kTile]; vsc[1] = sc[kTile + 8];
                if (tail) {
                    if (dead(slice0 + r8)) vsc[0] = 0.f;
                    if (dead(slice0 + r8 + 8)) vsc[1] = 0.f;
                }
            }
            if (Q8) {
                // a 16-byte chunk holds 16 dims: one ldmatrix.x4 feeds two k-steps
#pragma unroll
                for (int j = 0; j < HD / 32; ++j) {
                    const uint32_t chunk = (uint32_t)(2 * j + (mat >> 1));
                    const uint32_t addr = kst + k_rowoff + (((chunk & 7u) ^ k_sw) << 4);
                    uint32_t w0, w1, w2, w3;
                    ptx::ldmatrix_x4(addr, w0, w1, w2, w3);
                    w0 ^= 0x80808080u; w1 ^= 0x80808080u; w2 ^= 0x80808080u; w3 ^= 0x80808080u;
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const uint32_t lo = hh ? w2 : w0, hi = hh ? w3 : w1;  // keys 0-7 / keys 8-15 of the slice
                        const uint32_t a0 = q8_pair_biased(lo, 0x4140), a1 = q8_pair_biased(hi, 0x4140);
                        const uint32_t a2 = q8_pair_biased(lo, 0x4342), a3 = q8_pair_biased(hi, 0x4342);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
                            ptx::mma_16816<BF>(s[nt][0], s[nt][1], s[nt][2], s[nt][3], a0, a1, a2, a3, qa[2 * j + hh][nt],
                                               qa[2 * j + hh][2 + nt], s[nt][0], s[nt][1], s[nt][2], s[nt][3]);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) s[nt][i] -= qoff[nt][i & 1];
            } else {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                const uint32_t chunk = (uint32_t)(2 * ks + (mat >> 1));
                const uint32_t addr = kst + k_rowoff + (chunk >> 3) * half_bytes + (((chunk & 7u) ^ k_sw) << 4);
                uint32_t a0, a1, a2, a3;
                ptx::ldmatrix_x4(addr, a0, a1, a2, a3);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    ptx::mma_16816<BF>(s[nt][0], s[nt][1], s[nt][2], s[nt][3], a0, a1, a2, a3, qa[ks][nt],
                                       qa[ks][2 + nt], s[nt][0], s[nt][1], s[nt][2], s[nt][3]);
            }
            }
            // ---- online softmax down the columns (base-2 domain). Fast path: nothing exceeds
            // the running column maxima (the usual case after the first tiles), so the
            // probabilities come straight from one FMA and one EX2 each; only when some
            // value does are the exact maxima reduced with shuffles and the state rescaled.
            uint32_t pb[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float t[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    t[i] = fmaf(s[nt][i], ksl[i >> 1], -m_run[nt][i & 1]);  // +inf while m_run is -inf
                    if (tail && dead(slice0 + r8 + 8 * (i >> 1))) t[i] = -INFINITY;
                }
                const bool exceeds = fmaxf(fmaxf(t[0], t[1]), fmaxf(t[2], t[3])) > 0.f;
                if (__any_sync(0xffffffffu, exceeds)) {
                    float v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        v[i] = s[nt][i] * ksl[i >> 1];
                        if (tail && dead(slice0 + r8 + 8 * (i >> 1))) v[i] = -INFINITY;
                    }
                    float mx0 = fmaxf(v[0], v[2]), mx1 = fmaxf(v[1], v[3]);
#pragma unroll
                    for (int sh = 4; sh < 32; sh <<= 1) {
                        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
                        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
                    }
                    const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);  // finite
                    const float al0 = ptx::ex2(m_run[nt][0] - mn0), al1 = ptx::ex2(m_run[nt][1] - mn1);
                    l_run[nt][0] *= al0;
                    l_run[nt][1] *= al1;
#pragma unroll
                    for (int j = 0; j < HD / 16; ++j) {
                        o[j][nt][0] *= al0; o[j][nt][2] *= al0;
                        o[j][nt][1] *= al1; o[j][nt][3] *= al1;
                    }
                    m_run[nt][0] = mn0;
                    m_run[nt][1] = mn1;
                    t[0] = v[0] - mn0; t[1] = v[1] - mn1; t[2] = v[2] - mn0; t[3] = v[3] - mn1;
                }
                const float p0 = ptx::ex2(t[0]), p1 = ptx::ex2(t[1]), p2 = ptx::ex2(t[2]), p3 = ptx::ex2(t[3]);
                l_run[nt][0] += p0 + p2;
                l_run[nt][1] += p1 + p3;
                // C fragment (key rows, head cols) -> B fragment (k = key, n = head)
                // (int8 pool: the V scale of the key goes into its probability; the row sums above do not see it)
                pb[nt][0] = ptx::movmatrix_trans(Pack2<PT>::pack(p0 * vsc[0], p1 * vsc[0]));  // keys 0-7 of the slice
                pb[nt][1] = ptx::movmatrix_trans(Pack2<PT>::pack(p2 * vsc[1], p3 * vsc[1]));  // keys 8-15
            }
            // ---- O^T += V^T.P^T : rows = 16 dims per tile, cols = heads
            if (Q8) {
                // The transposing load moves 16-bit units, i.e. pairs of neighbouring dims: a thread ends up
                // with dims (2e, 2e+1) of keys (2c, 2c+1), e = lane / 4. MMA row e then stands for dim 2e of
                // the 16-dim block and row e + 8 for dim 2e + 1; the accumulators are read out accordingly.
#pragma unroll
                for (int j2 = 0; j2 < HD / 32; ++j2) {
                    const uint32_t chunk = (uint32_t)(2 * j2 + (mat & 1));
                    const uint32_t addr = vst + v_rowoff + (((chunk & 7u) ^ v_sw) << 4);
                    uint32_t w0, w1, w2, w3;  // (keys 0-7, block 2j2) (keys 0-7, block 2j2+1) (keys 8-15, 2j2) (keys 8-15, 2j2+1)
                    ptx::ldmatrix_x4_trans(addr, w0, w1, w2, w3);
                    w0 ^= 0x80808080u; w1 ^= 0x80808080u; w2 ^= 0x80808080u; w3 ^= 0x80808080u;
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const uint32_t lo = hh ? w1 : w0, hi = hh ? w3 : w2;
                        const uint32_t a0 = q8_pair_to_h2(lo, 0x4240), a1 = q8_pair_to_h2(lo, 0x4341);
                        const uint32_t a2 = q8_pair_to_h2(hi, 0x4240), a3 = q8_pair_to_h2(hi, 0x4341);
                        const int j = 2 * j2 + hh;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
                            ptx::mma_16816<BF>(o[j][nt][0], o[j][nt][1], o[j][nt][2], o[j][nt][3], a0, a1, a2, a3, pb[nt][0],
                                               pb[nt][1], o[j][nt][0], o[j][nt][1], o[j][nt][2], o[j][nt][3]);
                    }
                }
            } else {
#pragma unroll
            for (int j = 0; j < HD / 16; ++j) {
                const uint32_t chunk = (uint32_t)(2 * j + (mat & 1));
                const uint32_t addr = vst + v_rowoff + (chunk >> 3) * half_bytes + (((chunk & 7u) ^ v_sw) << 4);
                uint32_t a0, a1, a2, a3;
                ptx::ldmatrix_x4_trans(addr, a0, a1, a2, a3);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    ptx::mma_16816<BF>(o[j][nt][0], o[j][nt][1], o[j][nt][2], o[j][nt][3], a0, a1, a2, a3, pb[nt][0],
                                       pb[nt][1], o[j][nt][0], o[j][nt][1], o[j][nt][2], o[j][nt][3]);
            }
            }
        }
        // release the stage to the producer
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&empty[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        if (GROUPS > 1) turn ^= 1;

        if (meta.flags & 2) {
            // ---- merge the eight warps' (m, l, acc) and write the item's partial rows.
            // Warp wq of group 1 and warp wq of group 0 hold fragments of identical layout:
            // group 1 parks its state in slot wq, group 0 folds it into its registers and
            // parks the sum, then all consumer threads reduce the four slots.
            float l_tot[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    float l = l_run[nt][i];
#pragma unroll
                    for (int sh = 4; sh < 32; sh <<= 1) l += __shfl_xor_sync(0xffffffffu, l, sh);
                    l_tot[nt][i] = l;
                }
            auto park = [&]() {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int g = 8 * nt + 2 * c4 + i;
                        if (r8 == 0) {
                            sML[(wq * GP + g) * 2 + 0] = m_run[nt][i];
                            sML[(wq * GP + g) * 2 + 1] = l_tot[nt][i];
                        }
                        float* ar = sAcc + (size_t)(wq * GP + g) * S::kAccStride;
#pragma unroll
                        for (int j = 0; j < HD / 16; ++j) {
                            ar[16 * j + dim_lo] = o[j][nt][i];
                            ar[16 * j + dim_hi] = o[j][nt][2 + i];
                        }
                    }
            };
            if (GROUPS > 1) {
                if (group == 1) park();
                ptx::named_bar_sync(1, kConsumers * 32);
            }
            if (group == 0) {
                if (GROUPS > 1) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int g = 8 * nt + 2 * c4 + i;
                        const float mb = sML[(wq * GP + g) * 2 + 0], lb = sML[(wq * GP + g) * 2 + 1];
                        const float M = fmaxf(m_run[nt][i], mb);
                        const float wa = (m_run[nt][i] == -INFINITY) ? 0.f : exp2f(m_run[nt][i] - M);
                        const float wb = (mb == -INFINITY) ? 0.f : exp2f(mb - M);
                        const float* ar = sAcc + (size_t)(wq * GP + g) * S::kAccStride;
#pragma unroll
                        for (int j = 0; j < HD / 16; ++j) {
                            o[j][nt][i] = o[j][nt][i] * wa + ar[16 * j + dim_lo] * wb;
                            o[j][nt][2 + i] = o[j][nt][2 + i] * wa + ar[16 * j + dim_hi] * wb;
                        }
                        l_tot[nt][i] = l_tot[nt][i] * wa + lb * wb;
                        m_run[nt][i] = M;
                    }
                __syncwarp();  // every lane has read slot wq before it is overwritten
                }
                park();
            }
            ptx::named_bar_sync(1, kConsumers * 32);
            const int tid = threadIdx.x;  // consumer threads come first
            const bool direct = P.out != nullptr && meta.ns == 1;  // the item is the whole pair: final rows
            T* outp = static_cast<T*>(P.out);
            const int ob = meta.pair / P.Hkv, ohkv = meta.pair - ob * P.Hkv;
            const int64_t orow0 = ((int64_t)ob * P.Hq + (int64_t)ohkv * P.G) * HD;  // decode: query row = request
            for (int idx = tid; idx < P.G * HD; idx += kConsumers * 32) {
                const int g = idx / HD, d = idx - g * HD;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < kGroupWarps; ++w) M = fmaxf(M, sML[(w * GP + g) * 2]);
                float L = 0.f, A = 0.f;
#pragma unroll
                for (int w = 0; w < kGroupWarps; ++w) {
                    const float mw = sML[(w * GP + g) * 2];
                    const float wt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
                    L += sML[(w * GP + g) * 2 + 1] * wt;
                    A += sAcc[(size_t)(w * GP + g) * S::kAccStride + d] * wt;
                }
                if (direct) {
                    outp[orow0 + idx] = Num<T>::from_f(A * (L > 0.f ? 1.f / L : 0.f));  // as the combine kernel rounds
                    continue;
                }
                const int64_t pr = (int64_t)meta.prow + g;
                P.pacc[pr * HD + d] = A;
                if (d == 0) {
                    P.pm[pr] = M * 0.6931471805599453f;  // back to the natural-log domain
                    P.pl[pr] = L;
                }
            }
            if (P.out != nullptr && meta.ns > 1) {
                // One of several items of its pair: count it; the last one to arrive merges them all
                // (maximum first, then the weighted sums: the result does not depend on the order).
                __threadfence();
                ptx::named_bar_sync(1, kConsumers * 32);
                if (tid == 0) {
                    const int prev = atomicAdd(P.pair_counter + meta.pair, 1);
                    const int last = prev == meta.ns - 1 ? 1 : 0;
                    if (last) P.pair_counter[meta.pair] = 0;  // for the next launch
                    reinterpret_cast<volatile int*>(sML)[kGroupWarps * GP * 2] = last;
                }
                ptx::named_bar_sync(1, kConsumers * 32);
                if (reinterpret_cast<volatile int*>(sML)[kGroupWarps * GP * 2]) {
                    __threadfence();
                    for (int idx = tid; idx < P.G * HD; idx += kConsumers * 32) {
                        const int g = idx / HD, d = idx - g * HD;
                        // four items at a time, every load of the group issued before the first use (one
                        // round trip to L2 per group; a pair is rarely cut more often than that)
                        float M = -INFINITY, L = 0.f, A = 0.f;
                        for (int s0 = 0; s0 < meta.ns; s0 += 4) {
                            float mw[4], lw[4], aw[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const bool in = s0 + k < meta.ns;
                                const int64_t pr = (int64_t)(meta.item0 + (in ? s0 + k : 0)) * P.G + g;
                                mw[k] = in ? __ldcg(P.pm + pr) : -INFINITY;
                                lw[k] = in ? __ldcg(P.pl + pr) : 0.f;
                                aw[k] = in ? __ldcg(P.pacc + pr * HD + d) : 0.f;
                            }
                            const float Mn = fmaxf(fmaxf(M, fmaxf(mw[0], mw[1])), fmaxf(mw[2], mw[3]));
                            const float keep = (M == -INFINITY) ? 0.f : expf(M - Mn);
                            L *= keep; A *= keep;
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float wt = (mw[k] == -INFINITY) ? 0.f : expf(mw[k] - Mn);
                                L = fmaf(lw[k], wt, L);
                                A = fmaf(aw[k], wt, A);
                            }
                            M = Mn;
                        }
                        outp[orow0 + idx] = Num<T>::from_f(A * (L > 0.f ? 1.f / L : 0.f));  // as the combine kernel rounds
                    }
                }
            }
            ptx::named_bar_sync(1, kConsumers * 32);  // merge buffers free for the next item
        }
    }
}

// ---- host side ---------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int encode_tiled_16bit(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    cuuint64_t d[5], st[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; ++i) { d[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) st[i] = strides_bytes[i];
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, st, bx, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)r;
}

int encode_rows_map_3d(CUtensorMap* map, const void* base, uint64_t rows, uint32_t row_elems, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    const cuuint64_t dims[3] = {64, rows, row_elems / 64};
    const cuuint64_t strides[2] = {(cuuint64_t)row_elems * 2, 128};  // bytes, dims 1 and 2
    const cuuint32_t box[3] = {64, box_rows, row_elems / 64};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Plain 2-D view [rows, row_elems] with a {64, box_rows} box (one 128-byte half per copy),
// used when the driver refuses the 3-D view above.
static int encode_rows_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint32_t row_elems,
                              uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    const cuuint64_t dims[2] = {row_elems, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_elems * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)r;
}

// int8 pool: [rows, 128] bytes, one 128-byte line per key row, {128, box_rows} boxes.
static int encode_rows_map_u8(CUtensorMap* map, const void* base, uint64_t rows, uint32_t row_bytes, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {row_bytes, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)r;
}

static bool box_rows_ok(int64_t bs) {
    if (bs >= 64) return bs % 64 == 0;
    return bs >= 8 && 64 % bs == 0;
}

// Everything but the shape of the batch: dtype, head sizes, pages, alignment.
bool decode_mma_shape_ok(const RfxPagedAttentionArgs* a) {
    if (a->force_generic) return false;
    if (a->dtype != RFX_BF16 && a->dtype != RFX_F16) return false;
    if (a->head_dim != 128 && a->head_dim != 64) return false;
    if (a->kv_int8 && (a->head_dim != 128 || ((uintptr_t)a->k_scales % 16) || ((uintptr_t)a->v_scales % 16)))
        return false;  // an int8 row has to be one 128-byte line
    const int64_t G = a->num_q_heads / a->num_kv_heads;
    if (G > 16) return false;
    if ((G * a->head_dim * 2) % 16) return false;  // bulk copies move multiples of 16 bytes
    if (!box_rows_ok(a->block_size)) return false;
    if (((uintptr_t)a->k_cache % 16) || ((uintptr_t)a->v_cache % 16) || ((uintptr_t)a->q % 16)) return false;
    if (a->rope_cos && (((uintptr_t)a->rope_cos % 16) || ((uintptr_t)a->rope_sin % 16))) return false;
    if (a->num_blocks * a->num_kv_heads * a->block_size >= (1ll << 31)) return false;
    return true;
}

bool decode_mma_supported(const RfxPagedAttentionArgs* a) {
    if (a->q_start != nullptr || a->max_q_len > 1) return false;  // one query row per request
    return decode_mma_shape_ok(a);
}

int decode_mma_ctas(const RfxPagedAttentionArgs*) { return sm_count(); }

template <typename T, int HD, int GP, int STAGES, int GROUPS = 1, bool Q8 = false>
static int launch_decode_t(const RfxPagedAttentionArgs* a, const CUtensorMap& km, const CUtensorMap& vm,
                           const DecodeParams& P) {
    using S = DecodeSmem<HD, GP, STAGES, Q8>;
    static_assert(S::total <= 232448, "decode kernel shared memory exceeds the sm_100 per-CTA limit");
    auto kern = decode_mma_kernel<T, HD, GP, STAGES, GROUPS, Q8>;
    static PerDeviceOnce attr_set;  // per instantiation
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set.done(dev)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::total);
        if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "decode smem opt-in (%zu B): %s", S::total, cudaGetErrorString(e));
        attr_set.mark(dev);
    }
    cudaError_t le = launch_pdl(kern, dim3(decode_mma_ctas(a)), dim3((kGroupWarps * GROUPS + kProducers) * 32), S::total,
                                as_stream(a->stream), km, vm, P);
    if (le != cudaSuccess) return fail(RFX_CUDA_ERROR, "decode kernel launch: %s", cudaGetErrorString(le));
    return check_launch("rfx_paged_attention (decode MMA kernel)");
}

int launch_decode_mma(const RfxPagedAttentionArgs* a, const PlanLayout&, const PlanPtrs& Pp, bool single_row_requests_only,
                      bool merge_in_kernel) {
    const int HD = (int)a->head_dim;
    const int G = (int)(a->num_q_heads / a->num_kv_heads);
    const int R = (int)(a->block_size < 64 ? a->block_size : 64);
    CUtensorMap km, vm;
    const uint64_t rows = (uint64_t)(a->num_blocks * a->num_kv_heads * a->block_size);
    int map2d = (debug_flags() & kDbgTma2d) ? 1 : 0;  // the 2-D maps: a debugging aid
    int r1 = 0, r2 = 0;
    if (a->kv_int8) {
        map2d = 0;
        r1 = encode_rows_map_u8(&km, a->k_cache, rows, (uint32_t)HD, (uint32_t)R);
        r2 = encode_rows_map_u8(&vm, a->v_cache, rows, (uint32_t)HD, (uint32_t)R);
        if (r1 || r2) return fail(RFX_CUDA_ERROR, "cuTensorMapEncodeTiled (int8 pool) failed (%d, %d)", r1, r2);
    } else if (!map2d) {
        r1 = encode_rows_map_3d(&km, a->k_cache, rows, (uint32_t)HD, (uint32_t)R);
        r2 = encode_rows_map_3d(&vm, a->v_cache, rows, (uint32_t)HD, (uint32_t)R);
        if (r1 || r2) map2d = 1;
    }
    if (map2d && !a->kv_int8) {
        r1 = encode_rows_map_2d(&km, a->k_cache, rows, (uint32_t)HD, (uint32_t)R);
        r2 = encode_rows_map_2d(&vm, a->v_cache, rows, (uint32_t)HD, (uint32_t)R);
        if (r1 || r2) return fail(RFX_CUDA_ERROR, "cuTensorMapEncodeTiled failed (%d, %d)", r1, r2);
    }

    DecodeParams P;
    P.q = a->q; P.block_table = a->block_table;
    P.q_start = single_row_requests_only ? a->q_start : nullptr;
    P.rcos = a->rope_cos; P.rsin = a->rope_sin; P.rpos = a->rope_positions;
    P.hdr = Pp.hdr; P.part_first = Pp.part_first; P.items = Pp.items; P.item_prow = Pp.item_prow;
    P.pm = Pp.m; P.pl = Pp.l; P.pacc = Pp.acc;
    P.num_blocks = a->num_blocks; P.max_blocks = a->max_blocks; P.bt_sb = a->bt_stride_b;
    P.table_rows = a->table_rows;
    P.Hq = (int)a->num_q_heads; P.Hkv = (int)a->num_kv_heads; P.G = G;
    P.block_size = (int)a->block_size; P.box_rows = R; P.rope_inter = a->rope_interleaved;
    P.scale_log2 = a->sm_scale * 1.4426950408889634f;
    P.map2d = map2d;
    P.k_scales = a->kv_int8 ? a->k_scales : nullptr;
    P.v_scales = a->kv_int8 ? a->v_scales : nullptr;
    const bool merge = merge_in_kernel && !single_row_requests_only && a->out != nullptr;
    P.out = merge ? a->out : nullptr;
    P.pair_item_begin = Pp.pair_item_begin;
    P.pair_counter = Pp.pair_counter;
    P.n_pairs = (int)(a->batch * a->num_kv_heads);
    P.late_trigger = single_row_requests_only ? 1 : 0;
    if (a->kv_int8) {
        // half the bytes per stage: ten (eight) stages fit where the 16-bit pool has six (five)
        if (a->dtype == RFX_BF16) {
            if (G <= 8) return launch_decode_t<__nv_bfloat16, 128, 8, 10, 2, true>(a, km, vm, P);
            return launch_decode_t<__nv_bfloat16, 128, 16, 8, 1, true>(a, km, vm, P);
        }
        if (G <= 8) return launch_decode_t<__half, 128, 8, 10, 2, true>(a, km, vm, P);
        return launch_decode_t<__half, 128, 16, 8, 1, true>(a, km, vm, P);
    }

#define RFX_DECODE_CASE(T)                                                                   \
    if (HD == 128) {                                                                         \
        if (G <= 8) return launch_decode_t<T, 128, 8, 6, 2>(a, km, vm, P);                   \
        return launch_decode_t<T, 128, 16, 5>(a, km, vm, P);                                 \
    } else {                                                                                 \
        if (G <= 8) return launch_decode_t<T, 64, 8, 8, 2>(a, km, vm, P);                    \
        return launch_decode_t<T, 64, 16, 8>(a, km, vm, P);                                  \
    }
    if (a->dtype == RFX_BF16) { RFX_DECODE_CASE(__nv_bfloat16) }
    RFX_DECODE_CASE(__half)
#undef RFX_DECODE_CASE
}

}  // namespace rfx
