// Prefill / chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA owns two query tiles of one (request, kv head): each tile is T consecutive query
// tokens times the G query heads that share the kv head, T*G <= 128 rows (row = one
// (token, head) pair), so a K/V tile is read once for the whole GQA group and for both tiles.
// Ten warps:
//   warps 0-3 / 4-7  softmax of tile a / tile b: thread r owns row r (TMEM lane r). Reads its
//              128 scores from TMEM in one go, keeps the row maximum and sum in registers
//              (no shuffles), writes P as bf16 back into the TMEM columns S occupied, and
//              rescales O in TMEM only when a row maximum grew by more than 2^8 (a stale
//              maximum is exact as long as the final 1/l uses the same reference).
//   warp 8     TMA producer: both Q tiles once, then K and V tiles of 128 keys, two stages each,
//              128-byte swizzle; one box per page, holding both 64-wide halves (one per tile for
//              dense K/V and for pages of 128 keys or more).
//   warp 9     MMA issuer: S_x = Q_x.K_j^T (8 x tcgen05.mma 128x128x16 from shared-memory
//              descriptors), O_x += P_x.V_j with P read from TMEM and V as an MN-major
//              shared-memory operand, in the fixed order [P_a.V, S_a'] [P_b.V, S_b'] ...: the two
//              tiles ping-pong, one tile's warps run their softmax while the tensor core works
//              for the other (two independent issuers fall into lock-step and lose that
//              overlap). A barrier poll by the issuing thread costs hundreds of cycles (it
//              competes with the tensor core's operand reads for shared memory), so the issuer
//              waits only for P_x ready, which also carries the producer's vote that V_j and
//              K_{j+1} have landed.
//              Completion through tcgen05.commit on mbarriers.
// TMEM: columns [0,128) S_a/P_a, [128,256) S_b/P_b, [256,384) O_a, [384,512) O_b (fp32).
//
// Shared-memory form of a K/V tile. Paged: [group of 8 keys][64-wide half][8 keys][128 B], i.e.
// 2 KiB per 8 keys, which is what one TMA box {64 elems, 8 keys, 2 halves, page/8 groups} of a
// 4-D view of the pool writes; the MMA descriptors walk it with 2 KiB between 8-key groups and
// 1 KiB between the halves. Dense: [half][128 keys][128 B] (1 KiB between groups, 16 KiB between
// halves). Both are 128-byte swizzled in 1 KiB atoms.
//
// Causal masking is bottom-right aligned: token t of n sees keys 0..ctx-n+t; K tiles wholly
// above the diagonal are never loaded. Tensor-pipe bound: 4*rows*keys*D FLOPs per tile pair.
//
// The way out. A thread owns a whole row, so rows stored straight from the threads put the 32 rows
// of every store instruction into 32 different lines. Whole rows (no split over the keys): a tile
// whose rows all have a query is written into its Q buffer in the Q box's layout and leaves as two
// TMA stores through a tensor map over the output; other tiles are stored row by row. Split over
// the keys: a warp's 32 partial rows are one 16 KB block of the workspace, passed through shared
// memory and stored 512 contiguous bytes per instruction.
//
// Split batches take their work from the plan's list of units -- (item, pair of query tiles), the
// longest first -- one CTA per unit; a CTA beyond the list leaves on one header read.
#include <stdlib.h>

#include <type_traits>

#include "paged_plan.cuh"
#include "ptx.cuh"

namespace rfx {

constexpr int kPfThreads = 320;
constexpr int kPfKeys = 128;          // keys per K/V tile
constexpr int kPfHD = 128;            // head_dim
constexpr int kPfHalfBytes = 128 * 128;  // one 64-wide half of a 128-row tile
constexpr int kPfTileBytes = 2 * kPfHalfBytes;
constexpr int kPfKvStages = 2;
constexpr float kPfRescaleTau = 8.0f;  // log2 units

struct PrefillParams {
    void* out;
    int64_t out_tok_stride, out_head_stride;  // elements
    const int64_t* block_table;                // paged K/V, or nullptr for dense
    const int32_t* ctx_lens;                   // [B] keys per request (paged)
    const int32_t* q_start;                    // [B+1] first query row per request (paged)
    int32_t* status;                           // optional device status word
    // split-K mode (items != nullptr): a CTA handles one plan item (request, kv head, key range)
    // and leaves un-normalised (m, l, acc) partial rows for the combine kernel
    const int4* items;
    const int32_t* item_prow;
    const int32_t* hdr;
    const int2* unit_order;
    float* pm;
    float* pl;
    float* pacc;
    int items_cap;
    int skip_single;                           // split-K mode: requests with one query row belong to the decode kernel
    int out_by_tma;                            // 1: `omap` covers the output (laid out like Q): whole tiles are stored through shared memory by TMA
    int wait_late;                             // 1: the kernel before this one (the decode kernel of a mixed batch) is waited for by the grid's last CTA only, at its end
    int64_t bt_sb, max_blocks, num_blocks;
    int B, Hq, Hkv, G, T;                      // T = query tokens per tile = 128 / G
    int Sq, Sk;                                // dense sizes (paged: Sq = host bound on rows per request)
    int block_size;
    int box_keys, box_shift, boxes_per_tile;   // keys per TMA box (a power of two), boxes per 128-key tile
    uint32_t kv_sbo, kv_half;                  // bytes between 8-key groups / between the 64-wide halves of a tile
    int n_qtiles;                              // CTAs per (request, kv head) = ceil(Sq / 2T)
    int head_major_rows;                       // 0: row = t*G + g (paged Q [N,Hq,D]); 1: row = g*T + t (dense [B,H,S,D])
    int causal;
    float scale_log2;
    // dense only: additive mask [B, Hq, Sq, Sk] in the tensors' type (nullptr: none); 1 / sm_scale
    const void* mask;
    float inv_scale;
};

struct PfSmem {
    static constexpr size_t off_q = 0;                                   // two query tiles
    static constexpr size_t off_k = 2 * (size_t)kPfTileBytes;
    static constexpr size_t off_v = off_k + (size_t)kPfKvStages * kPfTileBytes;
    static constexpr size_t off_bars = off_v + (size_t)kPfKvStages * kPfTileBytes;
    // barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pv_done[2], o_staged[2]
    static constexpr int n_bars = 1 + 4 * kPfKvStages + 8;
    static constexpr size_t off_misc = off_bars + 8 * n_bars;
    static constexpr size_t total = off_misc + 64 + 1024;  // misc: TMEM base, abort flag, 4 bad-box masks
};

enum PfBar { PF_QFULL = 0, PF_KFULL = 1, PF_KEMPTY = 3, PF_VFULL = 5, PF_VEMPTY = 7, PF_SFULL = 9, PF_PFULL = 11,
             PF_PVDONE = 13, PF_OSTAGED = 15 };

template <typename T, bool MASK>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                  const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap omap,
                  const PrefillParams P) {
    constexpr bool BF = std::is_same<T, __nv_bfloat16>::value;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* sQ = smem + PfSmem::off_q;
    unsigned char* sK = smem + PfSmem::off_k;
    unsigned char* sV = smem + PfSmem::off_v;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PfSmem::off_bars);
    uint32_t* misc = reinterpret_cast<uint32_t*>(smem + PfSmem::off_misc);  // [0] TMEM base, [1] abort flag
    volatile uint32_t* sbad = misc + 4;  // [4] boxes of K tile j (slot j % 4) that could not be loaded: bad page index

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Launched with programmatic stream serialisation. Normally everything before this kernel (the plan)
    // has to be complete before anything is read. In a mixed batch the kernel before this one is the decode
    // kernel for the one-row requests, which itself started only when the plan was complete and lets its
    // dependents start then: this kernel's CTAs take the SMs as that kernel's CTAs leave them. The grid
    // must not complete before that kernel has (the combine kernel behind reads both kernels' partial
    // rows), but a CTA that waited for it would hold its SM until then, so one CTA waits for all: the last
    // of the grid, at its end. The plan is read past L1 (this CTA may have started before the grid
    // boundary that would have emptied it).
    if (!P.wait_late) ptx::pdl_wait();
    ptx::pdl_trigger();
    const bool waiter = P.wait_late && blockIdx.x == gridDim.x - 1;

    // ---- which pair of tiles: the latest query tokens first (most K tiles under causal masking)
    int qt, b, hkv, kb = 0, ke_item = 0x7fffffff, prow = 0;
    if (P.items) {
        // the plan lists the units of work -- (item, pair of query tiles) -- the longest first
        if ((int)blockIdx.x >= __ldcg(&P.hdr[HdrNumUnits])) { if (waiter) ptx::pdl_wait(); return; }
        const int2 unit = __ldcg(&P.unit_order[blockIdx.x]);
        const int item = unit.x;
        qt = unit.y;
        const int4 d = __ldcg(&P.items[item]);
        b = d.x; hkv = d.y; kb = d.z; ke_item = d.w;
        prow = __ldcg(&P.item_prow[item]);
    } else {
        const int pairs = P.B * P.Hkv;
        qt = P.n_qtiles - 1 - (int)(blockIdx.x / pairs);
        const int pair = (int)(blockIdx.x % pairs);
        b = pair / P.Hkv; hkv = pair % P.Hkv;
    }
    const int q0 = P.q_start ? P.q_start[b] : 0;
    const int n_q = P.q_start ? (P.q_start[b + 1] - q0) : P.Sq;
    const int ctx = P.ctx_lens ? max(0, P.ctx_lens[b]) : P.Sk;
    const int tok0 = qt * 2 * P.T;                  // tile a: tok0.., tile b: tok0 + T..
    // Whole rows per CTA: the grid was sized from the host's bound on the rows of a request; rows
    // beyond it would silently keep stale output, so say so in the status word. (Split batches are
    // checked by the plan kernel.)
    if (!P.items && threadIdx.x == 0 && P.status && qt == P.n_qtiles - 1 && n_q > P.n_qtiles * 2 * P.T)
        atomicOr(P.status, kStatusCapacity);
    if (tok0 >= n_q || (P.skip_single && n_q == 1)) {  // uniform over the CTA; nothing allocated yet
        if (waiter) ptx::pdl_wait();
        return;
    }
    const int off = ctx - n_q;                      // bottom-right: token t sees keys <= t + off
    const int last_tok = min(n_q, tok0 + 2 * P.T) - 1;
    // keys [kb, kv_end) are streamed: the item's range cut at the causal bound of the last row
    const int kv_end = min(ke_item, P.causal ? max(0, min(ctx, last_tok + off + 1)) : ctx);
    const int n_kv = kv_end > kb ? (kv_end - kb + kPfKeys - 1) / kPfKeys : 0;
    const int n_tiles = (tok0 + P.T < n_q) ? 2 : 1;  // a short chunk leaves tile b without rows: it is not run

    if (threadIdx.x == 0) {
        for (int i = 0; i < PfSmem::n_bars; ++i)
            // P ready: the tile's 128 softmax threads and the producer's vote (see `landed`)
            // O staged: the tile's 128 softmax threads (see the epilogue)
            ptx::mbar_init(&bars[i], (i == PF_PFULL || i == PF_PFULL + 1) ? 129u : (i == PF_OSTAGED || i == PF_OSTAGED + 1) ? 128u : 1u);
        misc[1] = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 9) ptx::tmem_alloc(&misc[0], 512);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = misc[0];
    volatile uint32_t* abort_flag = &misc[1];

    auto give_up = [&]() {
        if (P.status) atomicOr(P.status, 1);
        *abort_flag = 1;
    };
    // Bounded wait. The abort flag is looked at only once the wait drags on: a shared-memory
    // load costs > 100 cycles while the tensor core streams operands.
    auto wait_phase = [&](int bar, uint32_t parity) -> bool {
        for (uint32_t i = 0; i < (1u << 22); ++i) {
            if (ptx::mbar_try_wait(&bars[bar], parity)) return true;
            if (i > 1024) {
                if (*abort_flag) return false;
                __nanosleep(32);
            }
        }
        return false;
    };

    // byte offset of key row r (0..127), 16-byte chunk c (0..15) inside a K/V tile (before swizzling,
    // which only permutes the eight chunks of one 128-byte line)
    auto kv_row_off = [&](int r, int c) -> uint32_t {
        return (uint32_t)(r >> 3) * P.kv_sbo + (uint32_t)(c >> 3) * P.kv_half + (uint32_t)(r & 7) * 128u +
               (uint32_t)(c & 7) * 16u;
    };

    if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer --
        if (lane == 0) {
            ptx::prefetch_tensormap(&qmap);
            ptx::prefetch_tensormap(&kmap);
            ptx::prefetch_tensormap(&vmap);
            // Q: two tiles x two 64-wide halves; rows beyond T*G stay stale and are never stored
            ptx::mbar_arrive_expect_tx(&bars[PF_QFULL], 2u * (uint32_t)n_tiles * (uint32_t)(P.T * P.G) * 128u);
            for (int x = 0; x < n_tiles; ++x)
                for (int h = 0; h < 2; ++h) {
                    unsigned char* dst = sQ + x * kPfTileBytes + h * kPfHalfBytes;
                    if (P.head_major_rows)
                        ptx::tma_load_3d(dst, &qmap, &bars[PF_QFULL], h * 64, tok0 + x * P.T, b * P.Hq + hkv * P.G);
                    else
                        ptx::tma_load_3d(dst, &qmap, &bars[PF_QFULL], h * 64, hkv * P.G, q0 + tok0 + x * P.T);
                }
        }
        const int R = P.box_keys;
        // The producer's vote on P_i ready (both tiles): V_i and K_{i+1} have landed. A barrier
        // poll costs a few hundred cycles while the tensor core streams operands from shared
        // memory, so it is kept out of the issuer's and the softmax warps' loops; this warp has
        // the time. Keys at or past kv_end carry probability zero but their V rows may hold NaN
        // patterns: cleared here, before the vote.
        auto landed = [&](int i) -> bool {
            int ok = 1;
            if (lane == 0) {
                ok = wait_phase(PF_VFULL + i % kPfKvStages, (uint32_t)((i / kPfKvStages) & 1)) ? 1 : 0;
                if (ok && i + 1 < n_kv)
                    ok = wait_phase(PF_KFULL + (i + 1) % kPfKvStages, (uint32_t)(((i + 1) / kPfKvStages) & 1)) ? 1 : 0;
                if (!ok) give_up();
            }
            if (!__shfl_sync(0xffffffffu, ok, 0)) return false;
            const int valid = kv_end - (kb + i * kPfKeys);
            if (valid < kPfKeys) {
                unsigned char* vt = sV + (size_t)(i % kPfKvStages) * kPfTileBytes;
                for (int i2 = lane; i2 < (kPfKeys - valid) * 16; i2 += 32)
                    *reinterpret_cast<uint4*>(vt + kv_row_off(valid + (i2 >> 4), i2 & 15)) = make_uint4(0, 0, 0, 0);
                ptx::fence_proxy_async_smem();
                __syncwarp();
            }
            if (lane == 0) {
                ptx::mbar_arrive(&bars[PF_PFULL + 0]);
                if (n_tiles == 2) ptx::mbar_arrive(&bars[PF_PFULL + 1]);
            }
            return true;
        };
        for (int j = 0; j < n_kv; ++j) {
            const int st = j % kPfKvStages;
            const uint32_t par = (uint32_t)((j / kPfKvStages) & 1);
            const int key0 = kb + j * kPfKeys;
            // lane i owns box i of the tile: its coordinates in the 4-D view
            int c1 = 0, c3 = -1;
            bool bad = false;
            if (lane < P.boxes_per_tile) {
                const int key = key0 + lane * R;
                if (key < kv_end) {
                    if (P.block_table) {
                        const int64_t lb = key / P.block_size;
                        const int64_t page = lb < P.max_blocks ? P.block_table[(int64_t)b * P.bt_sb + lb] : -1;
                        if (page >= 0 && page < P.num_blocks)
                            c3 = (int)(((page * P.Hkv + hkv) * P.block_size + (key - lb * P.block_size)) >> 3);
                        else
                            bad = true;
                    } else {
                        c1 = key;
                        c3 = b * P.Hkv + hkv;
                    }
                }
            }
            const unsigned have = __ballot_sync(0xffffffffu, c3 >= 0);
            const unsigned badm = __ballot_sync(0xffffffffu, bad);
            const uint32_t tx = (uint32_t)__popc(have) * (uint32_t)R * 256u;
            if (badm && lane == 0 && P.status) atomicOr(P.status, kStatusBadPage);
            for (int which = 0; which < 2; ++which) {  // 0: K, 1: V
                uint64_t* fullb = &bars[(which ? PF_VFULL : PF_KFULL) + st];
                unsigned char* tile = (which ? sV : sK) + (size_t)st * kPfTileBytes;
                int ok = 1;
                if (lane == 0) ok = wait_phase((which ? PF_VEMPTY : PF_KEMPTY) + st, par ^ 1u) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { if (lane == 0) give_up(); goto done; }
                if (badm) {
                    // a page index outside the pool: its keys are masked by the softmax warps (sbad) and
                    // its rows are cleared here, so that they count as absent, as in the scalar kernel
                    for (int i2 = lane; i2 < kPfKeys * 16; i2 += 32) {
                        const int r = i2 >> 4;
                        if ((badm >> (r >> P.box_shift)) & 1u)
                            *reinterpret_cast<uint4*>(tile + kv_row_off(r, i2 & 15)) = make_uint4(0, 0, 0, 0);
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                }
                if (lane == 0) {
                    if (!which) sbad[j & 3] = badm;  // a slot is reused only after the softmax of tile j + 1
                    ptx::mbar_arrive_expect_tx(fullb, tx);
                }
                __syncwarp();
                if (c3 >= 0)
                    ptx::tma_load_4d(tile + (size_t)lane * R * 256, which ? &vmap : &kmap, fullb, 0, c1, 0, c3);
            }
            if (j > 0 && !landed(j - 1)) goto done;
        }
        if (n_kv > 1) {
            // The vote for the last tile must not fall into the phase of the tile before it (inside
            // the loop the wait for a free V stage orders the votes): that phase is over once the
            // P.V of tile n_kv-2 has released its V stage, which is what a load of tile n_kv would
            // wait for.
            int ok = 1;
            if (lane == 0) {
                ok = wait_phase(PF_VEMPTY + n_kv % kPfKvStages, (uint32_t)(((n_kv / kPfKvStages) & 1) ^ 1)) ? 1 : 0;
                if (!ok) give_up();
            }
            if (!__shfl_sync(0xffffffffu, ok, 0)) goto done;
        }
        if (n_kv > 0 && !landed(n_kv - 1)) goto done;
    } else if (warp == 9) {
        // ------------------------------------------------------------------- MMA issuer --
        constexpr uint32_t idesc_s = ptx::umma_idesc_f16(128, 128, BF ? 1 : 0, 0, 0);   // Q, K both K-major
        constexpr uint32_t idesc_o = ptx::umma_idesc_f16(128, 128, BF ? 1 : 0, 0, 1);   // P (TMEM), V MN-major
        const uint32_t q_addr = ptx::smem_u32(sQ);
        // lane 0 waits, every lane learns the outcome
        auto wait_bar = [&](int bar, uint32_t parity) -> bool {
            int ok = 1;
            if (lane == 0) ok = wait_phase(bar, parity) ? 1 : 0;
            return __shfl_sync(0xffffffffu, ok, 0) != 0;
        };
        // descriptor halves: a byte offset inside a tile is a 32-bit add on the low word
        const uint32_t hi_q = ptx::umma_desc_hi(1024), hi_kv = ptx::umma_desc_hi(P.kv_sbo);
        const uint32_t q_lo0 = ptx::umma_desc_lo(q_addr, 16);
        const uint32_t k_lo0 = ptx::umma_desc_lo(ptx::smem_u32(sK), 16);
        const uint32_t v_lo0 = ptx::umma_desc_lo(ptx::smem_u32(sV), P.kv_half);
        const uint32_t half16 = P.kv_half >> 4, vstep = P.kv_sbo >> 3;  // 16 keys of V = two 8-key groups
        auto issue_s = [&](int x, int jj) {  // S_x = Q_x . K_jj^T
            if (lane == 0) {
                const uint32_t qlo = q_lo0 + (uint32_t)x * (kPfTileBytes >> 4);
                const uint32_t klo = k_lo0 + (uint32_t)(jj % kPfKvStages) * (kPfTileBytes >> 4);
                const uint32_t klo1 = klo + half16;
#pragma unroll
                for (int ks = 0; ks < kPfHD / 16; ++ks)
                    ptx::umma_ss_lh(tmem + x * 128, qlo + (uint32_t)((ks >> 2) * (kPfHalfBytes >> 4) + (ks & 3) * 2), hi_q,
                                    ((ks >> 2) ? klo1 : klo) + (uint32_t)((ks & 3) * 2), hi_kv, idesc_s, ks > 0 ? 1u : 0u);
                ptx::umma_commit(&bars[PF_SFULL + x]);
                if (x == n_tiles - 1) ptx::umma_commit(&bars[PF_KEMPTY + jj % kPfKvStages]);
            }
        };
        if (!wait_bar(PF_QFULL, 0)) { if (lane == 0) give_up(); goto done; }
        if (n_kv > 0) {
            if (!wait_bar(PF_KFULL + 0, 0)) { if (lane == 0) give_up(); goto done; }
            ptx::tc_fence_after_sync();
            issue_s(0, 0);
            if (n_tiles == 2) issue_s(1, 0);
        }
        for (int j = 0; j < n_kv; ++j) {
            const int st = j % kPfKvStages;
            // No waits for V_j and K_{j+1} here: the producer warp adds its vote to P_j ready only
            // when both have landed.
            for (int x = 0; x < n_tiles; ++x) {
                if (!wait_bar(PF_PFULL + x, (uint32_t)(j & 1))) { if (lane == 0) give_up(); goto done; }
                ptx::tc_fence_after_sync();
                if (lane == 0) {
                    const uint32_t vlo = v_lo0 + (uint32_t)st * (kPfTileBytes >> 4);
                    const uint32_t pa = tmem + x * 128, od = tmem + 256 + x * 128;
#pragma unroll
                    for (int ks = 0; ks < kPfKeys / 16; ++ks)
                        ptx::umma_ts_lh(od, pa + ks * 8, vlo + (uint32_t)ks * vstep, hi_kv, idesc_o,
                                        (j > 0 || ks > 0) ? 1u : 0u);
                    ptx::umma_commit(&bars[PF_PVDONE + x]);
                    if (x == n_tiles - 1) ptx::umma_commit(&bars[PF_VEMPTY + st]);
                }
                // next S for this tile right behind its P.V: the tensor pipe runs them in order,
                // so the new scores land only after P has been read
                if (j + 1 < n_kv) issue_s(x, j + 1);
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax warps --
        const int x = warp >> 2;                                // which query tile
        const int r = (warp & 3) * 32 + lane;                   // row of the tile = TMEM lane
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_base + x * 128;
        const uint32_t o_addr = lane_base + 256 + x * 128;
        const int rows_used = P.T * P.G;
        const int t_loc = P.head_major_rows ? (r % P.T) : (r / P.G);
        const int g = P.head_major_rows ? (r / P.T) : (r % P.G);
        const int tok = tok0 + x * P.T + t_loc;
        const bool row_live = r < rows_used && tok < n_q;
        // A warp without a live row only keeps the barriers going; a tile without one is not run.
        const bool warp_live = __any_sync(0xffffffffu, row_live);
        if (x >= n_tiles) goto done;
        // keys 0..last_key are visible to this row; -1 for a dead row masks everything
        const int last_key = row_live ? min(kv_end - 1, P.causal ? min(ctx - 1, tok + off) : ctx - 1) : -1;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok_all = true;
        for (int j = 0; j < n_kv && ok_all; ++j) {
            if (!__all_sync(0xffffffffu, wait_phase(PF_SFULL + x, (uint32_t)(j & 1)) ? 1 : 0)) {
                if (lane == 0) give_up();
                ok_all = false;
                break;
            }
            ptx::tc_fence_after_sync();
            if (!warp_live) {  // nothing to compute: P of these rows stays whatever S was, O rows are never read
                ptx::tc_fence_before_sync();
                ptx::mbar_arrive(&bars[PF_PFULL + x]);
                continue;
            }
            const int key0 = kb + j * kPfKeys;
            // rows without a query (stale Q, results never stored) take no mask and trigger no rescale
            const bool need_mask = row_live && key0 + kPfKeys - 1 > last_key;
            uint32_t v[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) ptx::tmem_ld32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
            const uint32_t badk = sbad[j & 3];  // almost always 0
            ptx::tmem_wait_ld();
            if (MASK) {
                // score * scale + mask = (score + mask / scale) * scale: the mask joins the raw scores, so
                // the rest of the tile's softmax is the unmasked code. One row of the mask per thread.
                if (row_live) {
                    const T* mrow = static_cast<const T*>(P.mask) +
                                    (((int64_t)b * P.Hq + hkv * P.G + g) * P.Sq + tok) * (int64_t)P.Sk + key0;
                    const int nk = min(kPfKeys, P.Sk - key0);
                    if (nk == kPfKeys && (reinterpret_cast<uintptr_t>(mrow) & 15) == 0) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const uint4 w = reinterpret_cast<const uint4*>(mrow)[c];
                            const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                v[c * 8 + i] = __float_as_uint(fmaf(Num<T>::to_f(e[i]), P.inv_scale, __uint_as_float(v[c * 8 + i])));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 128; ++i)  // fully unrolled: v[] has to stay in registers
                            if (i < nk) v[i] = __float_as_uint(fmaf(Num<T>::to_f(mrow[i]), P.inv_scale, __uint_as_float(v[i])));
                    }
                }
            }
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (key0 + i > last_key) v[i] = 0xff800000u;  // -inf
            }
            if (badk) {
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if ((badk >> (i >> P.box_shift)) & 1u) v[i] = 0xff800000u;
            }
            // row maximum over four independent chains of three-input maxima
            float m4[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) m4[k] = fmaxf(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
#pragma unroll
            for (int i = 8; i < 128; i += 8) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    m4[k] = ptx::max3(m4[k], __uint_as_float(v[i + 2 * k]), __uint_as_float(v[i + 2 * k + 1]));
            }
            float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            mx *= P.scale_log2;  // scale > 0, so max and scale commute
            const bool grow = row_live && mx > m_run + kPfRescaleTau;  // also true for the first finite maximum
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = fmaxf(m_run, mx);
                const float alpha = (m_new == -INFINITY) ? 1.f : ptx::ex2(m_run - m_new);
                if (j > 0) {
                    // O holds tiles 0..j-1 once P.V of tile j-1 is done
                    if (!__all_sync(0xffffffffu,
                                    wait_phase(PF_PVDONE + x, (uint32_t)((j - 1) & 1)) ? 1 : 0)) {
                        if (lane == 0) give_up();
                        ok_all = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t w[32];
                        ptx::tmem_ld32(o_addr + c * 32, w);
                        ptx::tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) * alpha);
                        ptx::tmem_st32(o_addr + c * 32, w);
                    }
                    ptx::tmem_wait_st();
                }
                l_run *= alpha;
                m_run = m_new;
            }
            const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
            // probabilities, packed to 16 bits, written over the S columns (all already in registers)
            float2 ls[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};  // independent partial sums
            const float2 sc2 = make_float2(P.scale_log2, P.scale_log2), nm2 = make_float2(-m_use, -m_use);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    // two scores per FMA and per add (the packed fp32 forms)
                    const float2 t = __ffma2_rn(make_float2(__uint_as_float(v[c * 32 + i]), __uint_as_float(v[c * 32 + i + 1])), sc2, nm2);
                    const float p0 = ptx::ex2(t.x), p1 = ptx::ex2(t.y);
                    ls[(i >> 1) & 1] = __fadd2_rn(ls[(i >> 1) & 1], make_float2(p0, p1));
                    if (BF) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                        pk[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                    } else {
                        __half2 h = __floats2half2_rn(p0, p1);
                        pk[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                    }
                }
                ptx::tmem_st16(s_addr + c * 16, pk);
            }
            l_run += (ls[0].x + ls[0].y) + (ls[1].x + ls[1].y);
            ptx::tmem_wait_st();
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&bars[PF_PFULL + x]);
        }
        // ---- epilogue: O / l -> global
        if (ok_all && n_kv > 0) {
            if (!__all_sync(0xffffffffu, wait_phase(PF_PVDONE + x, (uint32_t)((n_kv - 1) & 1)) ? 1 : 0)) {
                if (lane == 0) give_up();
                ok_all = false;
            }
            ptx::tc_fence_after_sync();
        }
        if (ok_all && P.items) {
            // split-K: un-normalised partial of this row; the running maximum goes back to natural logs
            const int64_t pr = (int64_t)prow + (int64_t)tok * P.G + g;
            if (row_live) {
                P.pm[pr] = m_run * 0.6931471805599453f;
                P.pl[pr] = l_run;
            }
            // The accumulator rows: a thread's row is 512 contiguous bytes and the rows of a tile are
            // consecutive in the partial array, so the warp's 32 rows are one block of 16 KB. Written
            // straight from the threads, every store instruction touched 32 different lines (32 such
            // instructions per thread); instead the warp passes its block through shared memory -- 16 KB
            // of the Q buffers (tile a) or the K stages (tile b), all free since the last scores, 16-byte
            // pieces XOR-swizzled by the row so that neither side has bank conflicts -- and stores it
            // 512 contiguous bytes per instruction. Nothing crosses a warp: __syncwarp is all it needs.
            unsigned char* wbuf = (x == 0 ? sQ : sK) + (size_t)(warp & 3) * 16384;
            const int rl = r & 31;
            const int r_base = (warp & 3) * 32;
            const int live_rows = max(0, min(32, min(rows_used, (n_q - tok0 - x * P.T) * P.G) - r_base));
            if (n_kv > 0 && live_rows == 32 && P.out_by_tma) {
                // All 32 rows have a query: the block is written in the form of one TMA box of a view
                // [4 column blocks][rows][128 B] of the partial array (128-byte swizzle) and one thread
                // hands it over; the threads save their store and wait instructions.
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t w[32];
                    ptx::tmem_ld32(o_addr + c * 32, w);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<uint4*>(wbuf + c * 4096 + rl * 128 + ((i ^ (rl & 7)) << 4)) =
                            make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    ptx::tma_store_3d(&omap, wbuf, 0, (int)((int64_t)prow + (int64_t)(tok0 + x * P.T) * P.G + r_base), 0);
                    ptx::tma_store_commit();
                    ptx::tma_store_wait_read();
                }
            } else {
            if (n_kv > 0) {  // uniform over the CTA; the load is warp-collective
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t w[32];
                    ptx::tmem_ld32(o_addr + c * 32, w);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<uint4*>(wbuf + rl * 512 + (((c * 8 + i) ^ rl) << 4)) =
                            make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
                }
            }
            __syncwarp();
            float* gblock = P.pacc + ((int64_t)prow + (int64_t)(tok0 + x * P.T) * P.G + r_base) * kPfHD;
#pragma unroll 4
            for (int k = 0; k < live_rows; ++k) {
                const uint4 v = n_kv > 0 ? *reinterpret_cast<const uint4*>(wbuf + k * 512 + ((lane ^ k) << 4))
                                         : make_uint4(0, 0, 0, 0);
                reinterpret_cast<uint4*>(gblock + (size_t)k * kPfHD)[lane] = v;
            }
            }
        } else if (ok_all && P.out_by_tma && tok0 + x * P.T + P.T <= n_q) {
            // Every row of the tile has a query: the tile goes out the way Q came in. A thread's row is
            // 256 contiguous bytes, so the 32 rows of a warp's store instruction lie in 32 different
            // lines and sixteen such instructions per thread took 2 us per tile; here the rows are
            // written into the tile's Q buffer (free since the last scores), in the layout of the Q box
            // with its 128-byte swizzle, and one thread hands the two 64-wide halves to the TMA unit.
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            unsigned char* stile = sQ + (size_t)x * kPfTileBytes;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t w[32];
                if (n_kv > 0) {
                    ptx::tmem_ld32(o_addr + c * 32, w);
                    ptx::tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) w[i] = 0;
                }
                if (r < rows_used) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float a = __uint_as_float(w[i]) * inv, bq = __uint_as_float(w[i + 1]) * inv;
                        if (BF) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(a, bq);
                            pk[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                        } else {
                            __half2 h = __floats2half2_rn(a, bq);
                            pk[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                        }
                    }
                    // chunk c holds elements 32c .. 32c+31: half c/2, 16-byte pieces 4(c%2) .. 4(c%2)+3 of the row
                    unsigned char* hrow = stile + (size_t)(c >> 1) * kPfHalfBytes + (size_t)r * 128;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int piece = (c & 1) * 4 + i;
                        *reinterpret_cast<uint4*>(hrow + (((piece ^ (r & 7)) << 4))) =
                            make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                    }
                }
            }
            ptx::fence_proxy_async_smem();
            ptx::mbar_arrive(&bars[PF_OSTAGED + x]);
            if ((warp & 3) == 0 && lane == 0) {
                if (!wait_phase(PF_OSTAGED + x, 0)) {  // bounded like every wait: a warp that gave up never arrives
                    give_up();
                    goto done;
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (P.head_major_rows)
                        ptx::tma_store_3d(&omap, stile + h * kPfHalfBytes, h * 64, tok0 + x * P.T, b * P.Hq + hkv * P.G);
                    else
                        ptx::tma_store_3d(&omap, stile + h * kPfHalfBytes, h * 64, hkv * P.G, q0 + tok0 + x * P.T);
                }
                ptx::tma_store_commit();
                ptx::tma_store_wait_read();
            }
        } else if (ok_all) {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            T* orow = P.head_major_rows
                          ? reinterpret_cast<T*>(P.out) + (int64_t)tok * P.out_tok_stride +
                                (int64_t)(b * P.Hq + hkv * P.G + g) * P.out_head_stride
                          : reinterpret_cast<T*>(P.out) + (int64_t)(q0 + tok) * P.out_tok_stride +
                                (int64_t)(hkv * P.G + g) * P.out_head_stride;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t w[32];
                if (n_kv > 0) {
                    ptx::tmem_ld32(o_addr + c * 32, w);
                    ptx::tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) w[i] = 0;
                }
                if (row_live) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float a = __uint_as_float(w[i]) * inv, bq = __uint_as_float(w[i + 1]) * inv;
                        if (BF) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(a, bq);
                            pk[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                        } else {
                            __half2 h = __floats2half2_rn(a, bq);
                            pk[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
                        }
                    }
                    uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
                    for (int i = 0; i < 4; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                }
            }
        }
    }
done:
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 9) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, 512);
    }
    if (waiter) ptx::pdl_wait();
}

}  // namespace rfx

// ---- host side -------------------------------------------------------------------------
namespace rfx {

template <typename T, bool MASK = false>
static int launch_prefill_t(const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm,
                            const CUtensorMap& om, const PrefillParams& P, int grid, cudaStream_t stream) {
    auto kern = prefill_tc_kernel<T, MASK>;
    static PerDeviceOnce attr_set;  // per instantiation
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set.done(dev)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PfSmem::total);
        if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "prefill smem opt-in: %s", cudaGetErrorString(e));
        attr_set.mark(dev);
    }
    cudaError_t le = launch_pdl(kern, dim3(grid), dim3(kPfThreads), PfSmem::total, stream, qm, km, vm, om, P);
    if (le != cudaSuccess) return fail(RFX_CUDA_ERROR, "prefill_tc_kernel: %s", cudaGetErrorString(le));
    return check_launch("prefill_tc_kernel");
}

// Pages the K/V boxes can be cut from: whole groups of 8 keys, and either several pages per 128-key
// tile or several tiles per page.
static bool kv_box_ok(int64_t bs) { return bs >= 8 && ((bs <= kPfKeys && kPfKeys % bs == 0) || bs % kPfKeys == 0); }

static int log2_of(int v) {
    int s = 0;
    while ((1 << s) < v) ++s;
    return s;
}

// Dense fused_attention on tensor cores: q [B,H,Sq,D], k/v [B,Hkv,Sk,D]. Returns
// RFX_NOT_IMPLEMENTED for shapes the kernel does not cover (the caller then runs the scalar kernel).
bool dense_tensor_ok(const RfxAttentionArgs* a) {
    if (debug_flags() & kDbgNoTensorCore) return false;
    if (a->dtype != RFX_BF16 && a->dtype != RFX_F16) return false;
    if (a->head_dim != kPfHD) return false;
    if (a->attn_mask && !(a->sm_scale > 0.f)) return false;  // the mask is folded in as mask / scale
    const int G = (int)(a->num_q_heads / a->num_kv_heads);
    if (G > 128 || a->seq_k == 0) return false;
    if (a->seq_q * G < 32) return false;                 // decode-like: not worth a 128-row tile
    if (a->is_causal && a->seq_q != a->seq_k) return false;  // top-left causal on non-square
    if (((uintptr_t)a->q % 16) || ((uintptr_t)a->k % 16) || ((uintptr_t)a->v % 16) || ((uintptr_t)a->out % 16))
        return false;
    if (a->seq_k >= (1ll << 31) || a->seq_q >= (1ll << 31) || a->batch * a->num_q_heads >= (1ll << 31)) return false;
    return true;
}

int launch_dense_tensor(const RfxAttentionArgs* a) {
    if (!dense_tensor_ok(a)) return RFX_NOT_IMPLEMENTED;
    const int G = (int)(a->num_q_heads / a->num_kv_heads);
    const int T = 128 / G;
    CUtensorMap qm, km, vm, om;
    bool out_by_tma = false;
    {
        const uint64_t dims[3] = {(uint64_t)kPfHD, (uint64_t)a->seq_q, (uint64_t)(a->batch * a->num_q_heads)};
        const uint64_t str[2] = {(uint64_t)kPfHD * 2, (uint64_t)a->seq_q * kPfHD * 2};
        const uint32_t box[3] = {64, (uint32_t)T, (uint32_t)G};
        if (encode_tiled_16bit(&qm, a->q, 3, dims, str, box)) return RFX_NOT_IMPLEMENTED;
        out_by_tma = encode_tiled_16bit(&om, a->out, 3, dims, str, box) == 0;  // the output is laid out like Q
        if (!out_by_tma) om = qm;
    }
    {
        // [half][key][64 elems] per (batch, kv head): one box lands a whole 128-key tile, keys past
        // seq_k arrive as zeros
        const uint64_t dims[4] = {64, (uint64_t)a->seq_k, 2, (uint64_t)(a->batch * a->num_kv_heads)};
        const uint64_t str[3] = {(uint64_t)kPfHD * 2, 128, (uint64_t)a->seq_k * kPfHD * 2};
        const uint32_t box[4] = {64, (uint32_t)kPfKeys, 2, 1};
        if (encode_tiled_16bit(&km, a->k, 4, dims, str, box)) return RFX_NOT_IMPLEMENTED;
        if (encode_tiled_16bit(&vm, a->v, 4, dims, str, box)) return RFX_NOT_IMPLEMENTED;
    }
    PrefillParams P = {};
    P.out = a->out; P.out_tok_stride = kPfHD; P.out_head_stride = a->seq_q * kPfHD;
    P.block_table = nullptr; P.ctx_lens = nullptr; P.q_start = nullptr;
    P.status = (a->workspace && a->workspace_bytes >= 4) ? (int32_t*)a->workspace : nullptr;
    P.B = (int)a->batch; P.Hq = (int)a->num_q_heads; P.Hkv = (int)a->num_kv_heads; P.G = G; P.T = T;
    P.Sq = (int)a->seq_q; P.Sk = (int)a->seq_k;
    P.block_size = (int)a->seq_k; P.box_keys = kPfKeys; P.box_shift = 7; P.boxes_per_tile = 1;
    P.kv_sbo = 1024; P.kv_half = kPfKeys * 128;
    P.n_qtiles = (int)((a->seq_q + 2 * T - 1) / (2 * T));
    P.head_major_rows = 1; P.causal = a->is_causal;
    P.out_by_tma = out_by_tma ? 1 : 0;
    P.scale_log2 = a->sm_scale * 1.4426950408889634f;
    const int64_t grid = (int64_t)P.n_qtiles * P.B * P.Hkv;
    if (grid >= (1ll << 31)) return RFX_NOT_IMPLEMENTED;
    if (a->attn_mask) {
        P.mask = a->attn_mask;
        P.inv_scale = 1.0f / a->sm_scale;
        if (a->dtype == RFX_BF16)
            return launch_prefill_t<__nv_bfloat16, true>(qm, km, vm, om, P, (int)grid, as_stream(a->stream));
        return launch_prefill_t<__half, true>(qm, km, vm, om, P, (int)grid, as_stream(a->stream));
    }
    if (a->dtype == RFX_BF16) return launch_prefill_t<__nv_bfloat16>(qm, km, vm, om, P, (int)grid, as_stream(a->stream));
    return launch_prefill_t<__half>(qm, km, vm, om, P, (int)grid, as_stream(a->stream));
}

// Paged (chunked) prefill: q [N,Hq,D] already rotated, K/V in the pool.
bool prefill_paged_supported(const RfxPagedAttentionArgs* a) {
    if (a->force_generic || (debug_flags() & kDbgNoTensorCore)) return false;
    if (a->dtype != RFX_BF16 && a->dtype != RFX_F16) return false;
    if (a->kv_int8) return false;  // query chunks over an int8 pool run the scalar kernel
    if (a->head_dim != kPfHD || a->rope_cos) return false;
    if (a->q_start == nullptr || a->max_q_len < 1) return false;
    const int64_t G = a->num_q_heads / a->num_kv_heads;
    if (G > 128 || !kv_box_ok(a->block_size)) return false;
    if (((uintptr_t)a->q % 16) || ((uintptr_t)a->k_cache % 16) || ((uintptr_t)a->v_cache % 16) || ((uintptr_t)a->out % 16))
        return false;
    if (a->num_blocks * a->num_kv_heads * a->block_size >= (1ll << 34)) return false;  // box coordinate = row / 8
    return true;
}

// Split-K over the plan's items pays when the query chunks are short (a CTA per (request, kv
// head, tile pair) would otherwise stream a whole context, however uneven the contexts are).
// It needs key ranges that start on a K/V box boundary: items start at multiples of 64 keys.
bool prefill_paged_split(const RfxPagedAttentionArgs* a) {
    if (a->target_chunk < 0 || (debug_flags() & kDbgPrefillNoSplit)) return false;
    return a->block_size <= kPlanTile && kPlanTile % a->block_size == 0 && a->max_q_len <= 512;
}

// Runs per launch: CTAs of up to ~27 steps keep the last wave short (measured on the mixed
// batch: 1x 0.547, 2x 0.479, 3x 0.453, 4x 0.449, 6x 0.464 ms; a CTA costs ~6-11 us to start and finish).
// Runs the key stream of a split batch is cut into. With the units taken longest first and the one-row
// requests on the decode kernel, two per SM balance as well as more (cfg5: 1 x 0.330 ms, 2 x 0.330, 3 x
// 0.335, 4 x 0.347, 6 x 0.370, 8 x 0.401): every cut costs a CTA's set-up, a tile of partial rows written
// and read again, and a Q load.
int prefill_paged_parts(const RfxPagedAttentionArgs* a) { (void)a; return 2 * sm_count(); }
int prefill_paged_unit_rows(const RfxPagedAttentionArgs* a) { return 2 * (int)(128 / (a->num_q_heads / a->num_kv_heads)); }

// A request with a single query row fills 1/18th or less of a 128-row tile and still pays the
// tile's step time (about 64 KB of K/V per 4600 cycles and SM, a quarter of HBM speed). In a split
// batch such decode rows go to the decode kernel, which streams K/V at HBM speed; it runs first, this
// kernel's CTAs take the SMs its CTAs leave, and both leave partials for the one combine. Without
// one-row requests (the plan says so in the header) the decode kernel returns at once. The debug words
// mixed=0 / mixed=1 override the choice.
bool prefill_paged_mixed(const RfxPagedAttentionArgs* a) {
    if (!prefill_paged_split(a) || !decode_mma_shape_ok(a)) return false;
    if (debug_flags() & (kDbgMixedOn | kDbgMixedOff)) return (debug_flags() & kDbgMixedOn) != 0;
    return true;
}

int launch_prefill_paged(const RfxPagedAttentionArgs* a, int32_t* status_word, const PlanLayout* L,
                         const PlanPtrs* split, bool skip_single_row_requests) {
    const int G = (int)(a->num_q_heads / a->num_kv_heads);
    const int T = 128 / G;
    const int R = (int)(a->block_size < kPfKeys ? a->block_size : kPfKeys);  // keys per box
    CUtensorMap qm, km, vm, om;
    bool out_by_tma = false;
    {
        const uint64_t dims[3] = {(uint64_t)kPfHD, (uint64_t)a->num_q_heads, (uint64_t)a->n_q};
        const uint64_t str[2] = {(uint64_t)kPfHD * 2, (uint64_t)a->num_q_heads * kPfHD * 2};
        const uint32_t box[3] = {64, (uint32_t)G, (uint32_t)T};
        int r = encode_tiled_16bit(&qm, a->q, 3, dims, str, box);
        if (r) return fail(RFX_CUDA_ERROR, "cuTensorMapEncodeTiled(q) failed (%d)", r);
        // whole rows per CTA: the output [N, Hq, D] is laid out like Q
        out_by_tma = split == nullptr && encode_tiled_16bit(&om, a->out, 3, dims, str, box) == 0;
        if (!out_by_tma) om = qm;
    }
    if (split) {
        // the partial accumulator rows [cap_rows][128 fp32] seen as [4 column blocks][rows][64 16-bit units]
        const uint64_t dims[3] = {64, (uint64_t)L->cap_rows, 4};
        const uint64_t str[2] = {(uint64_t)kPfHD * 4, 128};
        const uint32_t box[3] = {64, 32, 4};
        out_by_tma = encode_tiled_16bit(&om, split->acc, 3, dims, str, box) == 0;
        if (!out_by_tma) om = qm;
    }
    {
        // The pool's rows (page, kv head, position) in groups of 8: [group][half][row in group][64 elems],
        // so one box {64, 8, 2, R/8} brings both halves of up to 128 keys of a page and lands them as
        // 2 KiB per group, halves 1 KiB apart.
        const uint64_t rows = (uint64_t)(a->num_blocks * a->num_kv_heads * a->block_size);
        const uint64_t dims[4] = {64, 8, 2, rows / 8};
        const uint64_t str[3] = {(uint64_t)kPfHD * 2, 128, 8ull * kPfHD * 2};
        const uint32_t box[4] = {64, 8, 2, (uint32_t)(R / 8)};
        int r1 = encode_tiled_16bit(&km, a->k_cache, 4, dims, str, box);
        int r2 = encode_tiled_16bit(&vm, a->v_cache, 4, dims, str, box);
        if (r1 || r2) return fail(RFX_CUDA_ERROR, "cuTensorMapEncodeTiled(kv) failed (%d, %d)", r1, r2);
    }
    PrefillParams P = {};
    P.out = a->out; P.out_tok_stride = a->num_q_heads * kPfHD; P.out_head_stride = kPfHD;
    P.block_table = a->block_table; P.ctx_lens = a->context_lens; P.q_start = a->q_start;
    P.status = status_word;
    P.bt_sb = a->bt_stride_b; P.max_blocks = a->max_blocks; P.num_blocks = a->num_blocks;
    P.B = (int)a->batch; P.Hq = (int)a->num_q_heads; P.Hkv = (int)a->num_kv_heads; P.G = G; P.T = T;
    P.Sq = (int)a->max_q_len; P.Sk = 0;
    P.block_size = (int)a->block_size; P.box_keys = R; P.box_shift = log2_of(R); P.boxes_per_tile = kPfKeys / R;
    P.kv_sbo = 2048; P.kv_half = 1024;
    P.n_qtiles = (int)((a->max_q_len + 2 * T - 1) / (2 * T));
    P.head_major_rows = 0; P.causal = a->is_causal;
    P.out_by_tma = out_by_tma ? 1 : 0;
    P.scale_log2 = a->sm_scale * 1.4426950408889634f;
    int64_t grid = (int64_t)P.n_qtiles * P.B * P.Hkv;
    if (split) {
        P.items = split->items; P.item_prow = split->item_prow; P.hdr = split->hdr; P.unit_order = split->unit_order;
        P.pm = split->m; P.pl = split->l; P.pacc = split->acc;
        // the plan makes at most one item per pair plus one per run boundary
        int64_t cap = a->batch * a->num_kv_heads + (a->target_chunk > 0 ? L->max_parts : prefill_paged_parts(a));
        if (cap > L->max_items) cap = L->max_items;
        P.items_cap = (int)cap;
        P.skip_single = skip_single_row_requests ? 1 : 0;
        P.wait_late = P.skip_single;  // then the decode kernel runs right before this one
        grid = (int64_t)P.n_qtiles * cap;
        if (grid > L->max_units) grid = L->max_units;  // the plan lists no more than that
    }
    if (grid >= (1ll << 31)) return fail(RFX_INVALID_ARGUMENT, "prefill grid too large");
    if (a->dtype == RFX_BF16) return launch_prefill_t<__nv_bfloat16>(qm, km, vm, om, P, (int)grid, as_stream(a->stream));
    return launch_prefill_t<__half>(qm, km, vm, om, P, (int)grid, as_stream(a->stream));
}

}  // namespace rfx
