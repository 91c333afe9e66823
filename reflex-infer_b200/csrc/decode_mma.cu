// Paged GQA decode, split-K partial kernel for 16-bit KV with head_dim 128 or 64.
//
// HBM-bound: every (request, kv_head, key-range) item streams its K and V pages exactly
// once. A persistent CTA per SM runs one producer warp and four consumer warps:
//   producer : pulls items from an atomic work counter, reads block-table entries 32 at a
//              time, and issues one TMA tile copy per page for K and for V into a ring of
//              64-key stages; each copy lands the page as [half][row][128 B] with the
//              128-byte swizzle, completion counted on the stage's mbarrier;
//   consumers: each takes 16 of the stage's 64 keys: S = Q.K^T with the G query heads of
//              the group as the (padded) 16 MMA rows, online softmax with quad shuffles,
//              O += P.V, all through m16n8k16 warp MMAs fed by conflict-free ldmatrix;
//              at the item's last stage the four warps merge (m, l, acc) through shared
//              memory and write one partial.
// RoPE can be fused into the Q load with torch's per-op rounding.
//
// Algorithmic bytes per item: 2 * keys * D * e (K and V). Arithmetic is G FLOP/byte, far
// below what the warp MMA path sustains, so the kernel's roofline is HBM bandwidth.
#include <stdlib.h>

#include <type_traits>

#include "paged_plan.cuh"
#include "ptx.cuh"

namespace rfx {

constexpr int kTile = 64;           // keys per stage
constexpr int kConsumers = 4;       // consumer warps, 16 keys each
constexpr int kDecodeThreads = (kConsumers + 1) * 32;
constexpr int kAccPad = 8;          // floats of padding per merge row (bank spread)

struct StageMeta {
    int item;      // -1: no more work
    int b, hkv;
    int n_valid;   // keys of this stage that exist (0..64)
    int flags;     // bit0 first stage of item, bit1 last stage of item
    int prow;      // first partial row of the item
    int pad0, pad1;
};

struct DecodeParams {
    const void* q;
    const int64_t* block_table;
    const void* rcos;
    const void* rsin;
    const int32_t* rpos;
    int32_t* hdr;
    const int4* items;
    const int32_t* item_prow;
    float* pm;
    float* pl;
    float* pacc;
    int64_t num_blocks, max_blocks, bt_sb, table_rows;
    int Hq, Hkv, G, block_size, box_rows, rope_inter;
    int map2d;         // 1: the maps are 2-D [rows, D] with {64, box_rows} boxes, one copy per 128-byte half
    float scale_log2;  // sm_scale * log2(e)
};

template <int HD, int GP, int STAGES>
struct DecodeSmem {
    static constexpr int kRowBytes = HD * 2;
    static constexpr int kTileBytes = kTile * kRowBytes;  // K or V of one stage
    static constexpr int kAccStride = HD + kAccPad;
    static constexpr size_t off_k = 0;
    static constexpr size_t off_v = (size_t)STAGES * kTileBytes;
    static constexpr size_t off_merge = 2 * (size_t)STAGES * kTileBytes;
    static constexpr size_t merge_bytes = (size_t)kConsumers * GP * kAccStride * 4;
    static constexpr size_t off_ml = off_merge + merge_bytes;             // [warps][GP][2]
    static constexpr size_t off_meta = off_ml + (size_t)kConsumers * GP * 2 * 4;
    static constexpr size_t off_bars = off_meta + (size_t)STAGES * sizeof(StageMeta);
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
    uint32_t r;
    uint16_t lo = *reinterpret_cast<uint16_t*>(&a), hi = *reinterpret_cast<uint16_t*>(&b);
    r = (uint32_t)lo | ((uint32_t)hi << 16);
    return r;
}

// Loads (and optionally rotates) the A fragments of Q for the item's G heads.
// qa[ks][0] = row g,   dims 16ks + 2c + {0,1};   qa[ks][1] = row g+8, same dims;
// qa[ks][2] = row g,   dims 16ks + 8 + 2c + ..;  qa[ks][3] = row g+8      (c = lane % 4).
template <typename T, int HD, int GP>
__device__ inline void load_q_frags(uint32_t (&qa)[HD / 16][4], const DecodeParams& P, int b, int hkv) {
    const int lane = threadIdx.x & 31;
    const int g0 = lane >> 2, c = lane & 3;
    const T* qb = (const T*)P.q + ((int64_t)b * P.Hq + (int64_t)hkv * P.G) * HD;
    const bool rope = P.rcos != nullptr;
    int64_t pos = 0;
    bool pos_ok = false;
    if (rope) {
        pos = P.rpos[b];
        pos_ok = pos >= 0 && pos < P.table_rows;
    }
    const T* cr = (const T*)P.rcos + (pos_ok ? pos : 0) * HD;
    const T* sr = (const T*)P.rsin + (pos_ok ? pos : 0) * HD;
#pragma unroll
    for (int rr = 0; rr < (GP > 8 ? 2 : 1); ++rr) {
        const int g = g0 + 8 * rr;
        const bool live = g < P.G;
        const T* qr = qb + (int64_t)g * HD;
        if (!rope || !pos_ok) {
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
        } else if (P.rope_inter) {
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
}

template <typename T, int HD, int GP, int STAGES>
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_mma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  const DecodeParams P) {
    using S = DecodeSmem<HD, GP, STAGES>;
    constexpr bool BF = std::is_same<T, __nv_bfloat16>::value;
    extern __shared__ unsigned char smem_raw[];
    // TMA's 128-byte swizzle is a function of the shared-memory address, so tiles must
    // start on 1024-byte boundaries; the launch asks for 1 KiB of slack.
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* sK = smem + S::off_k;
    unsigned char* sV = smem + S::off_v;
    float* sAcc = reinterpret_cast<float*>(smem + S::off_merge);
    float* sML = reinterpret_cast<float*>(smem + S::off_ml);
    StageMeta* sMeta = reinterpret_cast<StageMeta*>(smem + S::off_meta);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::off_bars);
    uint64_t* empty = full + STAGES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = P.box_rows;                 // rows per TMA box = min(block_size, 64)
    const uint32_t box_bytes = (uint32_t)R * S::kRowBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], kConsumers);
        }
        ptx::fence_barrier_init();
    }
    __syncthreads();

    if (warp == kConsumers) {
        // ------------------------------------------------------------ producer --
        if (lane == 0) {
            ptx::prefetch_tensormap(&kmap);
            ptx::prefetch_tensormap(&vmap);
        }
        const int n_items = P.hdr[HdrNumItems];
        int stage = 0;
        uint32_t phase = 0;
        bool alive = true;
        // Two-deep item pipeline: `cur` is being issued, `nxt_id` is known, the atomic for
        // the one after is in flight.
        int cur_id = 0, nxt_id = 0;
        if (lane == 0) {
            cur_id = atomicAdd(P.hdr + HdrWorkCounter, 1);
            nxt_id = atomicAdd(P.hdr + HdrWorkCounter, 1);
        }
        cur_id = __shfl_sync(0xffffffffu, cur_id, 0);
        nxt_id = __shfl_sync(0xffffffffu, nxt_id, 0);
        int4 cur = make_int4(0, 0, 0, 0);
        int cur_prow = 0;
        if (cur_id < n_items) { cur = P.items[cur_id]; cur_prow = P.item_prow[cur_id]; }
        while (alive && cur_id < n_items) {
            int4 nxt = make_int4(0, 0, 0, 0);
            int nxt_prow = 0;
            if (nxt_id < n_items) { nxt = P.items[nxt_id]; nxt_prow = P.item_prow[nxt_id]; }
            int nn_id = 0;
            if (lane == 0) nn_id = atomicAdd(P.hdr + HdrWorkCounter, 1);

            const int b = cur.x, hkv = cur.y, kb = cur.z, ke = cur.w;
            const int n_tiles = (ke - kb + kTile - 1) / kTile;
            const int64_t* bt = P.block_table + (int64_t)b * P.bt_sb;
            // window of 32 consecutive logical blocks held one per lane
            int win0 = kb / P.block_size;
            auto load_win = [&](int w0) -> int64_t {
                const int64_t lb = (int64_t)w0 + lane;
                const int64_t last = ((int64_t)ke - 1) / P.block_size;
                return (lb <= last && lb < P.max_blocks) ? bt[lb] : -1;
            };
            int64_t pg_cur = (n_tiles > 0) ? load_win(win0) : -1;
            int64_t pg_nxt = (n_tiles > 0) ? load_win(win0 + 32) : -1;
            const int it_count = n_tiles > 0 ? n_tiles : 1;  // an empty item still sends one stage
            for (int t = 0; t < it_count && alive; ++t) {
                const int tok0 = kb + t * kTile;
                const int n_valid = max(0, min(kTile, ke - tok0));
                const int n_boxes = (n_valid + R - 1) / R;
                bool ok = true;
                if (lane == 0) ok = ptx::mbar_wait_bounded(&empty[stage], phase ^ 1u);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
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
                if (lane == 0) {
                    StageMeta m;
                    m.item = cur_id; m.b = b; m.hkv = hkv; m.n_valid = n_valid;
                    m.flags = (t == 0 ? 1 : 0) | (t == it_count - 1 ? 2 : 0);
                    m.prow = cur_prow; m.pad0 = 0; m.pad1 = 0;
                    sMeta[stage] = m;
                    if (okmask != wantmask) atomicOr(P.hdr + HdrStatus, kStatusBadPage);
                    ptx::mbar_arrive_expect_tx(&full[stage], 2u * box_bytes * (uint32_t)__popc(okmask));
                }
                __syncwarp();
                if (lane < n_boxes && page_ok) {
                    const int row = (int)((my_page * P.Hkv + hkv) * P.block_size + my_row0);
                    unsigned char* kd = sK + (size_t)stage * S::kTileBytes + (size_t)lane * box_bytes;
                    unsigned char* vd = sV + (size_t)stage * S::kTileBytes + (size_t)lane * box_bytes;
                    if (!P.map2d) {
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
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                // advance the block window once the next stage starts beyond it
                const int next_lb = (tok0 + kTile) / P.block_size;
                if (next_lb - win0 >= 32 && t + 1 < it_count) {
                    win0 += 32;
                    pg_cur = pg_nxt;
                    pg_nxt = load_win(win0 + 32);
                }
            }
            cur_id = nxt_id; cur = nxt; cur_prow = nxt_prow;
            nxt_id = __shfl_sync(0xffffffffu, nn_id, 0);
        }
        // Tell the consumers there is nothing left.
        if (alive) {
            bool ok = true;
            if (lane == 0) ok = ptx::mbar_wait_bounded(&empty[stage], phase ^ 1u);
            if (lane == 0) {
                if (ok) {
                    StageMeta m;
                    m.item = -1; m.b = 0; m.hkv = 0; m.n_valid = 0; m.flags = 0; m.prow = 0; m.pad0 = 0; m.pad1 = 0;
                    sMeta[stage] = m;
                    ptx::mbar_arrive(&full[stage]);
                } else {
                    atomicOr(P.hdr + HdrStatus, kStatusWaitExpired);
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers --
    const int g0 = lane >> 2, c4 = lane & 3;
    uint32_t qa[HD / 16][4];
    float o[HD / 8][GP > 8 ? 4 : 2];
    float m_run[GP > 8 ? 2 : 1], l_run[GP > 8 ? 2 : 1];
    constexpr int NR = GP > 8 ? 2 : 1;

    // lane-constant parts of the ldmatrix addresses
    const int mat = lane >> 3, rowi = lane & 7;
    const int k_tok = warp * 16 + (mat >> 1) * 8 + rowi;  // K: matrices 0,1 keys 0-7; 2,3 keys 8-15
    const int v_tok = warp * 16 + (mat & 1) * 8 + rowi;   // V: matrices 0,2 keys 0-7; 1,3 keys 8-15
    const int k_box = k_tok / R, k_r = k_tok - k_box * R;
    const int v_box = v_tok / R, v_r = v_tok - v_box * R;
    const uint32_t k_rowoff = (uint32_t)k_box * box_bytes + (uint32_t)k_r * 128u;
    const uint32_t v_rowoff = (uint32_t)v_box * box_bytes + (uint32_t)v_r * 128u;
    const uint32_t half_bytes = (uint32_t)R * 128u;
    const uint32_t k_sw = (uint32_t)(k_r & 7), v_sw = (uint32_t)(v_r & 7);
    const uint32_t sK_u32 = ptx::smem_u32(sK), sV_u32 = ptx::smem_u32(sV);

    int stage = 0;
    uint32_t phase = 0;
    while (true) {
        // every lane acquires the stage itself; the vote keeps an expired wait warp-uniform
        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(&full[stage], phase) ? 1 : 0)) {
            if (lane == 0) atomicOr(P.hdr + HdrStatus, kStatusWaitExpired);
            break;
        }
        const StageMeta meta = sMeta[stage];
        if (meta.item < 0) break;
        if (meta.flags & 1) {
            load_q_frags<T, HD, GP>(qa, P, meta.b, meta.hkv);
#pragma unroll
            for (int r = 0; r < NR; ++r) { m_run[r] = -INFINITY; l_run[r] = 0.f; }
#pragma unroll
            for (int nt = 0; nt < HD / 8; ++nt)
#pragma unroll
                for (int i = 0; i < 2 * NR; ++i) o[nt][i] = 0.f;
        }
        const int slice0 = warp * 16;
        if (slice0 < meta.n_valid) {
            const uint32_t kst = sK_u32 + (uint32_t)stage * S::kTileBytes;
            const uint32_t vst = sV_u32 + (uint32_t)stage * S::kTileBytes;
            const bool tail = meta.n_valid < slice0 + 16;
            if (tail) {
                // Keys past the end may hold anything (stale pages, NaN patterns): their
                // probabilities are zero but 0*NaN would poison P.V, so clear those V rows.
                unsigned char* vs = sV + (size_t)stage * S::kTileBytes;
                for (int i = lane; i < 16 * (S::kRowBytes / 16); i += 32) {
                    const int tk = slice0 + i / (S::kRowBytes / 16);
                    const int ch = i % (S::kRowBytes / 16);
                    if (tk >= meta.n_valid) {
                        const int bx = tk / R, rr = tk - bx * R;
                        *reinterpret_cast<uint4*>(vs + (size_t)bx * box_bytes + (size_t)(ch >> 3) * half_bytes +
                                                  (size_t)rr * 128 + (size_t)(ch & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
            }
            // ---- S = Q.K^T : rows = heads of the group, cols = this warp's 16 keys
            float s[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                const uint32_t chunk = (uint32_t)(2 * ks + (mat & 1));
                const uint32_t addr = kst + k_rowoff + (chunk >> 3) * half_bytes + (((chunk & 7u) ^ k_sw) << 4);
                uint32_t b0, b1, b2, b3;
                ptx::ldmatrix_x4(addr, b0, b1, b2, b3);
                ptx::mma_16816<BF>(s[0][0], s[0][1], s[0][2], s[0][3], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3],
                                   b0, b1, s[0][0], s[0][1], s[0][2], s[0][3]);
                ptx::mma_16816<BF>(s[1][0], s[1][1], s[1][2], s[1][3], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3],
                                   b2, b3, s[1][0], s[1][1], s[1][2], s[1][3]);
            }
            // ---- online softmax (base-2 domain), rows g0 (+8)
            uint32_t pa[4];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                float v[4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        float x = s[nt][2 * r + i] * P.scale_log2;
                        if (tail) {
                            const int tk = slice0 + nt * 8 + 2 * c4 + i;
                            if (tk >= meta.n_valid) x = -INFINITY;
                        }
                        v[nt * 2 + i] = x;
                    }
                float mx = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run[r], mx);  // finite: the slice has a valid key
                const float alpha = exp2f(m_run[r] - m_new);
                float p[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) p[i] = exp2f(v[i] - m_new);
                l_run[r] = l_run[r] * alpha + (p[0] + p[1] + p[2] + p[3]);
                m_run[r] = m_new;
#pragma unroll
                for (int nt = 0; nt < HD / 8; ++nt) { o[nt][2 * r] *= alpha; o[nt][2 * r + 1] *= alpha; }
                pa[r] = Pack2<T>::pack(p[0], p[1]);      // keys 0-7 of the slice
                pa[2 + r] = Pack2<T>::pack(p[2], p[3]);  // keys 8-15
            }
            if (NR == 1) { pa[1] = 0; pa[3] = 0; }
            // ---- O += P.V
#pragma unroll
            for (int j = 0; j < HD / 16; ++j) {
                const uint32_t chunk = (uint32_t)(2 * j + (mat >> 1));
                const uint32_t addr = vst + v_rowoff + (chunk >> 3) * half_bytes + (((chunk & 7u) ^ v_sw) << 4);
                uint32_t b0, b1, b2, b3;
                ptx::ldmatrix_x4_trans(addr, b0, b1, b2, b3);
                if (NR == 2) {
                    ptx::mma_16816<BF>(o[2 * j][0], o[2 * j][1], o[2 * j][2], o[2 * j][3], pa[0], pa[1], pa[2],
                                       pa[3], b0, b1, o[2 * j][0], o[2 * j][1], o[2 * j][2], o[2 * j][3]);
                    ptx::mma_16816<BF>(o[2 * j + 1][0], o[2 * j + 1][1], o[2 * j + 1][2], o[2 * j + 1][3], pa[0],
                                       pa[1], pa[2], pa[3], b2, b3, o[2 * j + 1][0], o[2 * j + 1][1],
                                       o[2 * j + 1][2], o[2 * j + 1][3]);
                } else {
                    float j2, j3;
                    ptx::mma_16816<BF>(o[2 * j][0], o[2 * j][1], j2, j3, pa[0], pa[1], pa[2], pa[3], b0, b1,
                                       o[2 * j][0], o[2 * j][1], 0.f, 0.f);
                    ptx::mma_16816<BF>(o[2 * j + 1][0], o[2 * j + 1][1], j2, j3, pa[0], pa[1], pa[2], pa[3], b2,
                                       b3, o[2 * j + 1][0], o[2 * j + 1][1], 0.f, 0.f);
                }
            }
        }
        // release the stage to the producer
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&empty[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }

        if (meta.flags & 2) {
            // ---- merge the four warps' (m, l, acc) and write the item's partial rows
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                float l = l_run[r];
                l += __shfl_xor_sync(0xffffffffu, l, 1);
                l += __shfl_xor_sync(0xffffffffu, l, 2);
                const int g = g0 + 8 * r;
                if (c4 == 0) {
                    sML[(warp * GP + g) * 2 + 0] = m_run[r];
                    sML[(warp * GP + g) * 2 + 1] = l;
                }
                float* ar = sAcc + (size_t)(warp * GP + g) * S::kAccStride;
#pragma unroll
                for (int nt = 0; nt < HD / 8; ++nt)
                    *reinterpret_cast<float2*>(ar + nt * 8 + 2 * c4) = make_float2(o[nt][2 * r], o[nt][2 * r + 1]);
            }
            ptx::named_bar_sync(1, kConsumers * 32);
            const int tid = threadIdx.x;  // 0..127
            for (int idx = tid; idx < P.G * HD; idx += kConsumers * 32) {
                const int g = idx / HD, d = idx - g * HD;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < kConsumers; ++w) M = fmaxf(M, sML[(w * GP + g) * 2]);
                float L = 0.f, A = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumers; ++w) {
                    const float mw = sML[(w * GP + g) * 2];
                    const float wt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
                    L += sML[(w * GP + g) * 2 + 1] * wt;
                    A += sAcc[(size_t)(w * GP + g) * S::kAccStride + d] * wt;
                }
                const int64_t pr = (int64_t)meta.prow + g;
                P.pacc[pr * HD + d] = A;
                if (d == 0) {
                    P.pm[pr] = M * 0.6931471805599453f;  // back to the natural-log domain
                    P.pl[pr] = L;
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
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
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

static bool box_rows_ok(int64_t bs) {
    if (bs >= 64) return bs % 64 == 0;
    return bs >= 8 && 64 % bs == 0;
}

bool decode_mma_supported(const RfxPagedAttentionArgs* a) {
    if (a->force_generic) return false;
    if (a->dtype != RFX_BF16 && a->dtype != RFX_F16) return false;
    if (a->head_dim != 128 && a->head_dim != 64) return false;
    if (a->q_start != nullptr || a->max_q_len > 1) return false;  // one query row per request
    const int64_t G = a->num_q_heads / a->num_kv_heads;
    if (G > 16) return false;
    if (!box_rows_ok(a->block_size)) return false;
    if (((uintptr_t)a->k_cache % 1024) || ((uintptr_t)a->v_cache % 1024) || ((uintptr_t)a->q % 4)) return false;
    if (a->num_blocks * a->num_kv_heads * a->block_size >= (1ll << 31)) return false;
    return true;
}

int decode_mma_ctas(const RfxPagedAttentionArgs*) { return sm_count(); }

template <typename T, int HD, int GP, int STAGES>
static int launch_decode_t(const RfxPagedAttentionArgs* a, const PlanPtrs& Pp, const CUtensorMap& km,
                           const CUtensorMap& vm, const DecodeParams& P) {
    using S = DecodeSmem<HD, GP, STAGES>;
    auto kern = decode_mma_kernel<T, HD, GP, STAGES>;
    static bool attr_set[64] = {};  // per instantiation and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::total);
        if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "decode smem opt-in (%zu B): %s", S::total, cudaGetErrorString(e));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    (void)Pp;
    kern<<<decode_mma_ctas(a), kDecodeThreads, S::total, as_stream(a->stream)>>>(km, vm, P);
    return check_launch("rfx_paged_attention (decode MMA kernel)");
}

int launch_decode_mma(const RfxPagedAttentionArgs* a, const PlanLayout&, const PlanPtrs& Pp) {
    const int HD = (int)a->head_dim;
    const int G = (int)(a->num_q_heads / a->num_kv_heads);
    const int R = (int)(a->block_size < 64 ? a->block_size : 64);
    CUtensorMap km, vm;
    const uint64_t rows = (uint64_t)(a->num_blocks * a->num_kv_heads * a->block_size);
    static int force_2d = -1;  // REFLEX_B200_TMA2D=1 selects the 2-D maps (debugging aid)
    if (force_2d < 0) {
        const char* e = getenv("REFLEX_B200_TMA2D");
        force_2d = (e && e[0] == '1') ? 1 : 0;
    }
    int map2d = force_2d;
    int r1 = 0, r2 = 0;
    if (!map2d) {
        r1 = encode_rows_map_3d(&km, a->k_cache, rows, (uint32_t)HD, (uint32_t)R);
        r2 = encode_rows_map_3d(&vm, a->v_cache, rows, (uint32_t)HD, (uint32_t)R);
        if (r1 || r2) map2d = 1;
    }
    if (map2d) {
        r1 = encode_rows_map_2d(&km, a->k_cache, rows, (uint32_t)HD, (uint32_t)R);
        r2 = encode_rows_map_2d(&vm, a->v_cache, rows, (uint32_t)HD, (uint32_t)R);
        if (r1 || r2) return fail(RFX_CUDA_ERROR, "cuTensorMapEncodeTiled failed (%d, %d)", r1, r2);
    }

    DecodeParams P;
    P.q = a->q; P.block_table = a->block_table;
    P.rcos = a->rope_cos; P.rsin = a->rope_sin; P.rpos = a->rope_positions;
    P.hdr = Pp.hdr; P.items = Pp.items; P.item_prow = Pp.item_prow;
    P.pm = Pp.m; P.pl = Pp.l; P.pacc = Pp.acc;
    P.num_blocks = a->num_blocks; P.max_blocks = a->max_blocks; P.bt_sb = a->bt_stride_b;
    P.table_rows = a->table_rows;
    P.Hq = (int)a->num_q_heads; P.Hkv = (int)a->num_kv_heads; P.G = G;
    P.block_size = (int)a->block_size; P.box_rows = R; P.rope_inter = a->rope_interleaved;
    P.scale_log2 = a->sm_scale * 1.4426950408889634f;
    P.map2d = map2d;

#define RFX_DECODE_CASE(T)                                                                   \
    if (HD == 128) {                                                                         \
        if (G <= 8) return launch_decode_t<T, 128, 8, 6>(a, Pp, km, vm, P);                  \
        return launch_decode_t<T, 128, 16, 5>(a, Pp, km, vm, P);                             \
    } else {                                                                                 \
        if (G <= 8) return launch_decode_t<T, 64, 8, 8>(a, Pp, km, vm, P);                   \
        return launch_decode_t<T, 64, 16, 8>(a, Pp, km, vm, P);                              \
    }
    if (a->dtype == RFX_BF16) { RFX_DECODE_CASE(__nv_bfloat16) }
    RFX_DECODE_CASE(__half)
#undef RFX_DECODE_CASE
}

}  // namespace rfx
