// Windowed single gather for windows of at most 64 keys, query-anchored orientation ("packed" schedule),
// sm_100a.  One kernel in two modes:
//
//   PQ_FWD   Y[i] = sum_{j,k} softmax_{(j,k)}(scale Q_i.R_j.S_k) Vr[j] o Vs[k], with the statistics m, l
//   PQ_DQ    dQ[i] = scale * sum_j R_j o (sum_k gA[j][k] S_k),  gA = P o (dP - delta_i),
//            dP[j][k] = (dY_i o Vr_j) . Vs_k,  P from the forward's statistics
//
// The operator is the one of sg_ring_fwd.cuh / sg_ring_bwd.cuh (reference: cuda/forward.cu:108-477,
// cuda/backward.cu:415-934 with ROLE = BWD_QUERY_ANCHOR; small-window schedules of the reference:
// cuda/shared_kv/shared_retained_fwd.cuh:25-611).  What changes is how a 128-row tensor-core tile is filled.
// With a window of W <= 64 keys one query owns only W of the 128 tile rows, so QB = 128 / W consecutive
// queries share a tile:
//
//   tile row (g, js), g < QB, js < W:   query i0 + g, key  ring_key_w(i0 + g, js)   (a W-slot ring per query)
//   tile column ks < 128:               key ring_key(i0 + QB - 1, ks)               (one 128-slot ring per CTA)
//
// A tile step advances QB queries: QB keys enter the column ring, and each row group replaces QB of its W
// rows.  Cell (g, js, ks) is live iff both keys are visible from query i0 + g; everything else is masked to
// an exact zero before it is used as an MMA operand.  Per (tile, head) the products are the same
// 128x128xD MMAs as in the ring kernels, so the cost per query falls by QB.
//
// Roles, tensor-memory layout (two heads in flight: buffer b holds X -> P or gA at b*256 and U / dP -> Ug
// at b*256 + 128) and hand-offs follow sg_ring_fwd.cuh; the differences are
//   * every E thread owns one tile row and therefore one query: maxima, sums and the output collapse are
//     taken per row group (W lanes) instead of over the CTA;
//   * the rows of entering keys are staged QB at a time (one TMA box per tensor) into a small ring of
//     recent keys, from which the S / Vs ring rows and the per-thread R / Vr registers are refreshed;
//   * in PQ_DQ mode the H warps build two Hadamard tiles (Q o R and dY o Vr), the score-shaped products
//     X and dP are committed together, and the S ring is read by both X (K-major) and Ug (MN-major), so
//     at a tile boundary the kept-back Ug product is issued before the ring rows change.
// Restrictions (the launcher falls back to the ring kernels otherwise): D = 128, at least four query
// heads per KV head (bounds how far the H warps run ahead of the E warps: the recent-key ring is four
// tiles deep), q_begin and the block length multiples of QB.
#pragma once

#include <cuda.h>

#include "sg_ring_common.cuh"

namespace sgpack {

using namespace sgring;

enum PackMode { PQ_FWD = 0, PQ_DQ = 1 };

// Key held by row slot js of the W-slot ring of query i: the unique index congruent to js (mod W) in (i - W, i].
template <int W>
__device__ __forceinline__ int ring_key_w(int i, int js) { return i - ((i - js) & (W - 1)); }

struct QParams {
    const __nv_bfloat16* Q;        // [B,Hq,N,D]
    const __nv_bfloat16* R;        // [B,Hkv,N,D]
    const __nv_bfloat16* S;
    const __nv_bfloat16* Vr;
    const __nv_bfloat16* Vs;
    const uint8_t* mask;           // [B,N,N] or null
    const uint32_t* mask_words;    // the same mask as packed words [B,N,ceil(N/32)], or null (takes precedence)
    // PQ_FWD outputs
    __nv_bfloat16* Y;              // [B,Hq,N,D]
    float* m;                      // [B,Hq,N]
    float* l;
    // PQ_DQ inputs / output
    const float* m_in;             // forward statistics
    const float* l_in;
    const float* delta;            // [B,Hq,N]  rowsum(dY o Y)
    __nv_bfloat16* dQ;             // [B,Hq,N,D]
    int B, Hq, Hkv, N, window, q_begin, block_len;
    int bnhd;                      // memory layout of the [B,H,N,D] operands: 0 as written, 1 [B,N,H,D] (RowAddr)
    __nv_bfloat16* Y_act;          // PQ_FWD: optional second output QuickGELU(Y), laid out like Y; or null
    float scale;
    int* status;
    // TMA descriptors with boxes of QB rows: Q (and dY) viewed as [B*Hq*N, D], R, Vr, S, Vs as [B*Hkv*N, D]
    CUtensorMap tmQ, tmdY, tmR, tmVr, tmS, tmVs;
};

enum QBar {
    QB_QP_FULL0 = 0, QB_QP_FULL1, QB_X_DONE0, QB_X_DONE1, QB_P_FULL0, QB_P_FULL1, QB_U_DONE0, QB_U_DONE1,
    QB_U_FREE0, QB_U_FREE1, QB_GT_FULL, QB_H_SYNC, QB_M_SYNC, QB_STAGE0, QB_STAGE1, QB_E_SYNC,
    QB_NEXT_READY0, QB_COUNT = QB_NEXT_READY0 + 4
};

constexpr int KEY_TILES = 4;      // depth of the recent-key ring, in tiles

template <int D, int W, int MODE>
struct QSmem {
    static constexpr int QBN = RING / W;                // queries per tile
    static constexpr int TILE = RING * D * 2;           // bytes of one [128][D] BF16 tile
    static constexpr int SK = KEY_TILES * QBN;          // rows of the recent-key ring per tensor
    static constexpr int OFF_S = 0;
    static constexpr int OFF_VS = TILE;
    static constexpr int OFF_QP = 2 * TILE;             // 2 buffers
    static constexpr int OFF_GT = 4 * TILE;             // PQ_DQ: 1 buffer
    static constexpr int OFF_QSTAGE = OFF_GT + (MODE == PQ_DQ ? TILE : 0);   // 2 stages x {Q (, dY)} x QBN rows
    static constexpr int STAGE_BYTES = (MODE == PQ_DQ ? 2 : 1) * QBN * D * 2;
    static constexpr int OFF_KEYS = OFF_QSTAGE + 2 * STAGE_BYTES;            // [4 tensors][SK][D]: R, Vr, S, Vs
    // per head parity, per 16-row unit: D output partials, then l (column half 0, 1), the group maximum, a live flag
    static constexpr int OFF_RED = OFF_KEYS + 4 * SK * D * 2;                // 2 x 8 units x (D + 4) floats
    static constexpr int OFF_MPART = OFF_RED + 2 * 8 * (D + 4) * 4;          // 2 x 16 floats: half-warp maxima
    static constexpr int OFF_BARS = OFF_MPART + 2 * 16 * 4;
    static constexpr int OFF_MISC = OFF_BARS + QB_COUNT * 8;                 // tmem slot (4) + fail flag (4)
    static constexpr int BYTES = OFF_MISC + 16;
    static constexpr int ALLOC = BYTES + 1024;
};

// Sum over the 16 lanes of each half-warp of 32 per-lane values given as 16 BF16 pairs (w[k] = values 2k, 2k + 1).
// Four exchange stages on the packed pairs (the partial sums are rounded to BF16 at each, like the first four stages
// of warp_transpose_sum_words); lane L ends up with the half-warp totals of values 2 (L & 15) and 2 (L & 15) + 1.
__device__ __forceinline__ void halfwarp_transpose_sum_words(uint32_t (&w)[16], int lane, float& r0, float& r1) {
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int k = 0; k < o; ++k) {
            const uint32_t send = up ? w[k] : w[k + o];
            const uint32_t keep = up ? w[k + o] : w[k];
            const uint32_t got = __shfl_xor_sync(0xFFFFFFFFu, send, o);
            __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&keep);
            __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&got);
            __nv_bfloat162 c = __hadd2(a, b);
            w[k] = *reinterpret_cast<uint32_t*>(&c);
        }
    }
    const float2 v = unpack_bf16x2(w[0]);
    r0 = v.x;
    r1 = v.y;
}

// Visibility of the 128 column slots for query i (window and optional mask row), as four ballot words;
// every lane of the calling warp gets the same words.  i_last names the ring position (the tile's last query).
__device__ __forceinline__ void column_visibility(const MaskRow mask_row, int i, int i_last, int window, int lane,
                                                  uint32_t (&vw)[4]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int key = ring_key(i_last, q * 32 + lane);
        bool v = key >= 0 && key <= i && key > i - window;
        if (v && mask_row.any()) v = mask_row.at(key);
        vw[q] = __ballot_sync(0xFFFFFFFFu, v);
    }
}

template <int D, int W, int MODE>
__global__ void __launch_bounds__(PIPE_THREADS, 1) sg_pack_q_kernel(const __grid_constant__ QParams p) {
    using L = QSmem<D, W, MODE>;
    constexpr bool DQ = MODE == PQ_DQ;
    constexpr int QBN = RING / W;        // queries (row groups) per tile
    constexpr int CH = D / 8;            // 16-byte chunks per row
    constexpr int DW = D / 2;            // packed bf16x2 words per row
    constexpr int HD = D / 2;            // output columns per E thread
    constexpr int SK = L::SK;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int E_REGS = 120, H_REGS = DQ ? 200 : 152, M_REGS = DQ ? 72 : 96;
    static_assert(8 * E_REGS + 4 * H_REGS + 4 * M_REGS <= 2048, "register file: 64K registers / 32 lanes");
    static_assert(D == 128, "packed schedule: D = 128 only");
    static_assert(W == 16 || W == 32 || W == 64, "packed schedule: 16, 32 or 64 row slots per query");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sS = smem + L::OFF_S;
    uint8_t* sVs = smem + L::OFF_VS;
    uint8_t* sQp = smem + L::OFF_QP;
    uint8_t* sGt = smem + L::OFF_GT;
    uint8_t* sStage = smem + L::OFF_QSTAGE;
    uint8_t* sKeys = smem + L::OFF_KEYS;
    float* sRed = reinterpret_cast<float*>(smem + L::OFF_RED);
    float* sMpart = reinterpret_cast<float*>(smem + L::OFF_MPART);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::OFF_MISC);
    volatile int* sFail = reinterpret_cast<volatile int*>(smem + L::OFF_MISC + 4);
    constexpr int KEY_PLANE = SK * D * 2;                 // bytes of one tensor's plane of the recent-key ring
    // planes: 0 R, 1 Vr, 2 S, 3 Vs
    auto key_row = [&](int plane, int key) { return sKeys + plane * KEY_PLANE + (key & (SK - 1)) * (D * 2); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.z, g = blockIdx.y;
    const int G = p.Hq / p.Hkv;
    const int q0 = p.q_begin + blockIdx.x * p.block_len;
    const int q1 = min(q0 + p.block_len, p.N);
    if (q0 >= q1) return;
    const int n_tiles = (q1 - q0) / QBN;                  // q0, q1 are multiples of QBN
    const bool is_h = warp >= 8 && warp < 12, is_mma = warp == 12;

    if (is_mma) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int x = 0; x < 2; ++x) {
            mbar_init(&bars[QB_QP_FULL0 + x], 4);
            mbar_init(&bars[QB_X_DONE0 + x], 1);
            mbar_init(&bars[QB_P_FULL0 + x], 8);
            mbar_init(&bars[QB_U_DONE0 + x], 1);
            mbar_init(&bars[QB_U_FREE0 + x], 8);
            mbar_init(&bars[QB_STAGE0 + x], 1);
        }
        mbar_init(&bars[QB_GT_FULL], 4);
        mbar_init(&bars[QB_H_SYNC], 4);
        for (int x = 0; x < KEY_TILES; ++x) mbar_init(&bars[QB_NEXT_READY0 + x], 1);
        mbar_init(&bars[QB_M_SYNC], 8);
        mbar_init(&bars[QB_E_SYNC], 8);
        fence_mbar_init();
        *sFail = 0;
    }

    const size_t kv_base = (static_cast<size_t>(b) * p.Hkv + g) * p.N;       // statistics-style row index of key 0
    const RowAddr kaddr{p.bnhd, p.Hkv, p.N, D};
    const size_t kstep = kaddr.step();                                       // elements from one key's row to the next
    const __nv_bfloat16* gR = p.R + kaddr.elem(kv_base);
    const __nv_bfloat16* gS = p.S + kaddr.elem(kv_base);
    const __nv_bfloat16* gVr = p.Vr + kaddr.elem(kv_base);
    const __nv_bfloat16* gVs = p.Vs + kaddr.elem(kv_base);
    const MaskView mask_b = mask_view(p.mask, p.mask_words, b, p.N);
    const int n_iter = n_tiles * G;
    auto row_at = [&](int i, int hh) {
        return (static_cast<size_t>(b) * p.Hq + (g * G + hh)) * p.N + i;
    };
    // Element offset of the row of (position i, head hh of this KV group) in Q, dY, Y, dQ, its tensor-map coordinates,
    // and the coordinates of a key's row (RowAddr describes the two layouts; here without its divisions).
    auto qoff_at = [&](int i, int hh) -> size_t {
        return p.bnhd ? ((static_cast<size_t>(b) * p.N + i) * p.Hq + (g * G + hh)) * D
                      : ((static_cast<size_t>(b) * p.Hq + (g * G + hh)) * p.N + i) * D;
    };
    auto q_tma = [&](int i, int hh, int& x, int& y) {
        if (p.bnhd) { x = (g * G + hh) * D; y = b * p.N + i; }
        else { x = 0; y = (b * p.Hq + (g * G + hh)) * p.N + i; }
    };
    auto k_tma = [&](int key, int& x, int& y) {
        if (p.bnhd) { x = g * D; y = b * p.N + key; }
        else { x = 0; y = static_cast<int>(kv_base) + key; }
    };
    const size_t qstep = p.bnhd ? static_cast<size_t>(p.Hq) * D : D;      // elements between consecutive positions of one head
    const float c2 = p.scale * LOG2E;

    // True when any query of the tile that starts at i0 has a visible pair.  Without a caller mask every
    // query sees at least itself.
    auto tile_has_work = [&](int i0) {
        if (!mask_b.any()) return true;
        uint32_t any = 0;
#pragma unroll 1
        for (int gg = 0; gg < QBN; ++gg) {
            uint32_t vw[4];
            column_visibility(mask_b.row(i0 + gg), i0 + gg, i0 + QBN - 1, p.window, lane, vw);
            any |= vw[0] | vw[1] | vw[2] | vw[3];
        }
        return any != 0;
    };

    uint32_t tmem_base = 0;
    auto cta_start_sync = [&]() {
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        tmem_base = *tmem_slot;
    };

    if (is_h) {
        // ================================================================== H warps
        reg_inc<H_REGS>();
        const int hslot = tid - PIPE_E_THREADS;          // tile row of this thread
        const int hg = hslot / W, hjs = hslot & (W - 1);
        uint32_t rR[DW];
        uint32_t rVr[DQ ? DW : 1];
        int kcur = ring_key_w<W>(q0 + hg, hjs);
        {   // initial fill.  Column rings (slot = this thread's index) hold the keys visible from the tile's last
            // query; the row registers hold this row's key; the first tile's entering keys also go to the
            // recent-key ring, from which the next tile's rows are refreshed.
            const int ckey = ring_key(q0 + QBN - 1, hslot);
            const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                uint4 s = z, vs = z, r = z, vr = z;
                if (ckey >= 0) {
                    s = __ldg(reinterpret_cast<const uint4*>(gS + static_cast<size_t>(ckey) * kstep) + c);
                    vs = __ldg(reinterpret_cast<const uint4*>(gVs + static_cast<size_t>(ckey) * kstep) + c);
                }
                if (kcur >= 0) {
                    r = __ldg(reinterpret_cast<const uint4*>(gR + static_cast<size_t>(kcur) * kstep) + c);
                    if (DQ) vr = __ldg(reinterpret_cast<const uint4*>(gVr + static_cast<size_t>(kcur) * kstep) + c);
                }
                *reinterpret_cast<uint4*>(sS + sw128_offset<RING>(hslot, c)) = s;
                *reinterpret_cast<uint4*>(sVs + sw128_offset<RING>(hslot, c)) = vs;
                rR[4 * c] = r.x; rR[4 * c + 1] = r.y; rR[4 * c + 2] = r.z; rR[4 * c + 3] = r.w;
                if (DQ) { rVr[4 * c] = vr.x; rVr[4 * c + 1] = vr.y; rVr[4 * c + 2] = vr.z; rVr[4 * c + 3] = vr.w; }
            }
            for (int x = hslot; x < 4 * QBN * CH; x += PIPE_H_THREADS) {
                const int plane = x / (QBN * CH), rem = x % (QBN * CH), kr = rem / CH, c = rem % CH;
                const __nv_bfloat16* base = plane == 0 ? gR : plane == 1 ? gVr : plane == 2 ? gS : gVs;
                const int key = q0 + kr;
                *reinterpret_cast<uint4*>(key_row(plane, key) + c * 16) =
                    __ldg(reinterpret_cast<const uint4*>(base + static_cast<size_t>(key) * kstep) + c);
            }
        }
        // Row staging by TMA, issued by one thread: the QB query rows (Q, and dY in the dQ mode) of iteration
        // `it`, and, when next_tile > 0, the rows of the QB keys that enter with that tile.
        auto h_stage = [&](int it, int qi, int qh, int next_tile) {
            if (hslot != 0) return;
            if (it >= 0) {
                uint64_t* bar = &bars[QB_STAGE0 + (it & 1)];
                uint8_t* dst = sStage + (it & 1) * L::STAGE_BYTES;
                mbar_arrive_expect_tx(bar, L::STAGE_BYTES);
                int x, y;
                q_tma(qi, qh, x, y);
                tma_load_2d(dst, &p.tmQ, x, y, bar);
                if (DQ) tma_load_2d(dst + QBN * D * 2, &p.tmdY, x, y, bar);
            }
            if (next_tile > 0) {
                uint64_t* bar = &bars[QB_NEXT_READY0 + ((next_tile - 1) & (KEY_TILES - 1))];     // tile 0 has no staged keys
                const int key = q0 + next_tile * QBN;
                int kx, krow;
                k_tma(key, kx, krow);
                mbar_arrive_expect_tx(bar, 4 * QBN * D * 2);
                tma_load_2d(key_row(0, key), &p.tmR, kx, krow, bar);
                tma_load_2d(key_row(1, key), &p.tmVr, kx, krow, bar);
                tma_load_2d(key_row(2, key), &p.tmS, kx, krow, bar);
                tma_load_2d(key_row(3, key), &p.tmVs, kx, krow, bar);
            }
        };
        fence_async_smem();
        cta_start_sync();
        h_stage(0, q0, 0, -1);
        constexpr int HB = 8;                 // staged chunks in flight per thread
        int n = 0, it = 0;
        bool ok = true;
#pragma unroll 1
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int i0 = q0 + t * QBN;
            const bool work = tile_has_work(i0);
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh, ++it) {
                const bool boundary = hh == 0 && t > 0;       // QB keys enter, QB of this row group's slots change
                if (warp == 8) {
                    ok = pipe_wait<true>(&bars[QB_STAGE0 + (it & 1)], (it >> 1) & 1, sFail, 13);
                    if (ok && boundary)
                        ok = pipe_wait<true>(&bars[QB_NEXT_READY0 + ((t - 1) & (KEY_TILES - 1))], ((t - 1) / KEY_TILES) & 1, sFail, 14);
                }
                warp_arrive(&bars[QB_H_SYNC], lane);
                ok = ok & pipe_wait<true>(&bars[QB_H_SYNC], it & 1, sFail, 10);
                if (!ok) break;
                if (boundary) {
                    const int knew = ring_key_w<W>(i0 + hg, hjs);
                    if (knew != kcur) {
                        kcur = knew;
                        const uint4* r4 = reinterpret_cast<const uint4*>(key_row(0, knew));
                        const uint4* v4 = reinterpret_cast<const uint4*>(key_row(1, knew));
#pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            const uint4 a = r4[c];
                            rR[4 * c] = a.x; rR[4 * c + 1] = a.y; rR[4 * c + 2] = a.z; rR[4 * c + 3] = a.w;
                            if (DQ) {
                                const uint4 v = v4[c];
                                rVr[4 * c] = v.x; rVr[4 * c + 1] = v.y; rVr[4 * c + 2] = v.z; rVr[4 * c + 3] = v.w;
                            }
                        }
                    }
                }
                if (it + 1 < n_iter) {
                    const bool last_head = hh + 1 == G;
                    h_stage(it + 1, last_head ? i0 + QBN : i0, last_head ? 0 : hh + 1,
                            (hh == 0 && t + 1 < n_tiles) ? t + 1 : -1);
                }
                const int qb = n & 1;
                const uint8_t* stage = sStage + (it & 1) * L::STAGE_BYTES;
                if (work) {
                    // Qp[n&1] was last read by the score MMAs of head n-2
                    if (n >= 2) ok = pipe_wait<true>(&bars[QB_X_DONE0 + qb], ((n >> 1) - 1) & 1, sFail, 11);
                    if (!ok) break;
                    uint8_t* dQp = sQp + qb * L::TILE;
                    const uint4* q4 = reinterpret_cast<const uint4*>(stage + hg * (D * 2));
#pragma unroll
                    for (int c0 = 0; c0 < CH; c0 += HB) {
                        uint4 q[HB];
#pragma unroll
                        for (int c = 0; c < HB; ++c) q[c] = q4[c0 + c];
#pragma unroll
                        for (int c = 0; c < HB; ++c) {
                            uint4 o;
                            o.x = mul_bf16x2(q[c].x, rR[4 * (c0 + c)]);
                            o.y = mul_bf16x2(q[c].y, rR[4 * (c0 + c) + 1]);
                            o.z = mul_bf16x2(q[c].z, rR[4 * (c0 + c) + 2]);
                            o.w = mul_bf16x2(q[c].w, rR[4 * (c0 + c) + 3]);
                            st_shared_v4(dQp + sw128_offset<RING>(hslot, c0 + c), o.x, o.y, o.z, o.w);
                        }
                    }
                }
                if (boundary) {
                    // The column-ring rows change key once every product that reads them is complete: the
                    // score-shaped products of head n-1 (their commit covers dP in the dQ mode) and, in the
                    // dQ mode, the Ug product of head n-1, which the MMA warp issues before this head's.
                    if (n >= 1) ok = pipe_wait<true>(&bars[QB_X_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail, 12);
                    if (DQ && ok && n >= 1)
                        ok = pipe_wait<true>(&bars[QB_U_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail, 15);
                    if (!ok) break;
                    constexpr int NPL = DQ ? 2 : 1;           // S (and Vs: in the forward the E warps own that ring)
#pragma unroll
                    for (int x = hslot; x < NPL * QBN * CH; x += PIPE_H_THREADS) {
                        const int pl = x / (QBN * CH), rem = x % (QBN * CH), kr = rem / CH, c = rem % CH;
                        const int key = i0 + kr;
                        uint8_t* tile = pl == 0 ? sS : sVs;
                        *reinterpret_cast<uint4*>(tile + sw128_offset<RING>(key & (RING - 1), c)) =
                            *reinterpret_cast<const uint4*>(key_row(pl == 0 ? 2 : 3, key) + c * 16);
                    }
                }
                if (work || boundary) fence_async_smem();
                if (work) {
                    warp_arrive(&bars[QB_QP_FULL0 + qb], lane);
                    if (DQ) {
                        // Gt (one buffer) was last read by the dP product of head n-1
                        if (n >= 1) ok = pipe_wait<true>(&bars[QB_X_DONE0 + ((n - 1) & 1)], ((n - 1) >> 1) & 1, sFail, 16);
                        if (!ok) break;
                        const uint4* y4 = reinterpret_cast<const uint4*>(stage + QBN * D * 2 + hg * (D * 2));
#pragma unroll
                        for (int c0 = 0; c0 < CH; c0 += HB) {
                            uint4 y[HB];
#pragma unroll
                            for (int c = 0; c < HB; ++c) y[c] = y4[c0 + c];
#pragma unroll
                            for (int c = 0; c < HB; ++c) {
                                uint4 o;
                                o.x = mul_bf16x2(y[c].x, rVr[DQ ? 4 * (c0 + c) : 0]);
                                o.y = mul_bf16x2(y[c].y, rVr[DQ ? 4 * (c0 + c) + 1 : 0]);
                                o.z = mul_bf16x2(y[c].z, rVr[DQ ? 4 * (c0 + c) + 2 : 0]);
                                o.w = mul_bf16x2(y[c].w, rVr[DQ ? 4 * (c0 + c) + 3 : 0]);
                                st_shared_v4(sGt + sw128_offset<RING>(hslot, c0 + c), o.x, o.y, o.z, o.w);
                            }
                        }
                        fence_async_smem();
                        warp_arrive(&bars[QB_GT_FULL], lane);
                    }
                    ++n;
                }
            }
        }
    } else if (warp >= 12) {
        reg_dec<M_REGS>();
        cta_start_sync();
        if (is_mma) {
        // ================================================================== MMA warp
        const uint32_t issuer = elect_one();
        const uint32_t idesc_x = make_idesc_bf16(RING, RING, 0, 0);
        const uint32_t idesc_u = make_idesc_bf16(RING, D, 0, 1);
        const uint64_t dQp = make_smem_desc(smem_u32(sQp), 16, 1024, SWIZZLE_128B);           // A, K-major
        const uint64_t dGt = make_smem_desc(smem_u32(sGt), 16, 1024, SWIZZLE_128B);           // A, K-major (dQ mode)
        const uint64_t dS = make_smem_desc(smem_u32(sS), 16, 1024, SWIZZLE_128B);             // B, K-major
        const uint64_t dVsK = make_smem_desc(smem_u32(sVs), 16, 1024, SWIZZLE_128B);          // B, K-major (dQ mode)
        const uint64_t dVsM = make_smem_desc(smem_u32(sVs), RING * 128, 1024, SWIZZLE_128B);  // B, MN-major (forward)
        const uint64_t dSM = make_smem_desc(smem_u32(sS), RING * 128, 1024, SWIZZLE_128B);    // B, MN-major (dQ mode)
        int n = 0;
        bool ok = true, u_pending = false;
        // U(m) = P(m) Vs  (forward)   or   Ug(m) = gA(m) S  (dQ mode).  The BF16 A operand sits in the score
        // columns: thread (row, half c) keeps its 32 packed columns at the start of its own 64.
        auto issue_u = [&](int m) {
            const int ub = m & 1;
            bool r = pipe_wait<true>(&bars[QB_P_FULL0 + ub], (m >> 1) & 1, sFail, 22);
            if (!DQ && r && m >= 2) r = pipe_wait<true>(&bars[QB_U_FREE0 + ub], ((m >> 1) - 1) & 1, sFail, 23);
            if (r) {
                tc_fence_after();
                const uint32_t tX = tmem_base + ub * 256, tU = tX + 128;
                const uint64_t dB = DQ ? dSM : dVsM;
#pragma unroll
                for (int kk = 0; kk < RING / 16; ++kk)
                    umma_ts_pred(tU, tX + 64u * (kk >> 2) + 8u * (kk & 3), dB + kk * (2048 / 16), idesc_u, kk > 0, issuer);
                umma_commit_pred(&bars[QB_U_DONE0 + ub], issuer);
            }
            return r;
        };
#pragma unroll 1
        for (int t = 0; t < n_tiles && ok; ++t) {
            const bool work = tile_has_work(q0 + t * QBN);
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh) {
                if (!work || (DQ && hh == 0)) {
                    // nothing follows that would carry the kept-back product, or (dQ mode, tile boundary) the S
                    // ring rows are about to change: issue it now
                    if (u_pending) { ok = issue_u(n - 1); u_pending = false; }
                    if (!work) continue;
                    if (!ok) break;
                }
                const int qb = n & 1;
                ok = pipe_wait<true>(&bars[QB_QP_FULL0 + qb], (n >> 1) & 1, sFail, 20);
                // X[qb] held P / gA of head n-2 until the U product of that head had read it
                if (ok && n >= 2) ok = pipe_wait<true>(&bars[QB_U_DONE0 + qb], ((n >> 1) - 1) & 1, sFail, 21);
                // dQ mode: dP lands where Ug of head n-2 was; the E warps must have taken that out
                if (DQ && ok && n >= 2) ok = pipe_wait<true>(&bars[QB_U_FREE0 + qb], ((n >> 1) - 1) & 1, sFail, 24);
                if (!ok) break;
                tc_fence_after();
                {
                    const uint32_t tX = tmem_base + qb * 256;
                    const uint64_t dA = dQp + qb * (L::TILE / 16);
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = (kk >> 2) * (RING * 128 / 16) + (kk & 3) * 2;
                        umma_ss_pred(tX, dA + off, dS + off, idesc_x, kk > 0, issuer);
                    }
                    if (DQ) {
                        ok = pipe_wait<true>(&bars[QB_GT_FULL], n & 1, sFail, 25);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int kk = 0; kk < D / 16; ++kk) {
                            const uint32_t off = (kk >> 2) * (RING * 128 / 16) + (kk & 3) * 2;
                            umma_ss_pred(tX + 128, dGt + off, dVsK + off, idesc_x, kk > 0, issuer);
                        }
                    }
                    umma_commit_pred(&bars[QB_X_DONE0 + qb], issuer);
                }
                if (u_pending) {
                    ok = issue_u(n - 1);
                    if (!ok) break;
                }
                u_pending = true;
                ++n;
            }
        }
        if (ok && u_pending) ok = issue_u(n - 1);
        __syncwarp();
        }
    } else {
        // ================================================================== E warps
        reg_dec<E_REGS>();
        cta_start_sync();
        const int slot = tid & (RING - 1);               // tensor-memory lane = tile row
        const int ch = tid >> 7;                          // column half of the scores / of the output
        const int quarter = warp & 3;
        const int eg = slot / W, ejs = slot & (W - 1);   // row group (query of the tile) and its row slot
        const int unit = quarter * 2 + (W == 16 ? (lane >> 4) : 0);     // 16-row unit this thread's sums go to
        const uint32_t tl = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        constexpr int VW = HD / 2;                        // packed words of this thread's half of a value row
        // the row operand of the output collapse: Vr (forward) or R (dQ mode), this thread's half of the row
        const __nv_bfloat16* gRow = DQ ? gR : gVr;
        uint32_t rVr[VW];
        int kcur = ring_key_w<W>(q0 + eg, ejs);
        {
            if (kcur >= 0) {
                const uint4* v4 = reinterpret_cast<const uint4*>(gRow + static_cast<size_t>(kcur) * kstep + ch * HD);
#pragma unroll
                for (int c = 0; c < VW / 4; ++c) {
                    const uint4 v = __ldg(v4 + c);
                    rVr[4 * c] = v.x; rVr[4 * c + 1] = v.y; rVr[4 * c + 2] = v.z; rVr[4 * c + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int c = 0; c < VW; ++c) rVr[c] = 0;
            }
        }
        // Second half of an epilogue, run when the next one starts (or at the end): sum the units of each
        // row group and write the QB output rows (and statistics) of head fin_m.
        bool fin_pending = false;
        int fin_m = 0;
        size_t fin_row = 0, fin_off = 0;   // statistics row and element offset of the tile's first query
        auto finish = [&]() {
            if (!fin_pending) return true;
            fin_pending = false;
            if (!pipe_wait<true>(&bars[QB_E_SYNC], fin_m & 1, sFail, 33)) return false;
            const float* red = sRed + (fin_m & 1) * 8 * (D + 4);
            constexpr int UPG = W / 16;                   // 16-row units per row group
            constexpr int USTEP = W == 16 ? 1 : 2;        // with 32 rows or more per group only even units are written
#pragma unroll 1
            for (int idx = tid; idx < QBN * D; idx += PIPE_E_THREADS) {
                const int gg = idx / D, d = idx % D;
                float y = 0.f, Lsum = 0.f;
#pragma unroll
                for (int u = 0; u < UPG; u += USTEP) {
                    const float* ru = red + (gg * UPG + u) * (D + 4);
                    y += ru[d];
                    Lsum += ru[D] + ru[D + 1];
                }
                const float* r0 = red + (gg * UPG) * (D + 4);
                const bool live = r0[D + 3] != 0.f && (DQ || Lsum > 0.f);
                const size_t row = fin_row + gg;
                const size_t at = fin_off + gg * qstep + d;
                if (DQ) {
                    p.dQ[at] = __float2bfloat16(live ? p.scale * y : 0.f);
                } else {
                    // a query without a visible pair: Y = 0, m = NEG_INF, l = 0 (cuda/common.cuh:24)
                    const float yv = live ? y / Lsum : 0.f;
                    p.Y[at] = __float2bfloat16(yv);
                    if (p.Y_act) p.Y_act[at] = __float2bfloat16(yv / (1.f + __expf(-1.702f * yv)));
                    if (d == 0) {
                        p.m[row] = live ? r0[D + 2] * p.scale : NEG_INF_F;
                        p.l[row] = live ? Lsum : 0.f;
                    }
                }
            }
            return true;
        };
        // Epilogue of head m, one head late:  out[g][d] = sum_{rows of group g} rowop[d] * U[row][d].
        auto epilogue = [&](int m, size_t row0, size_t off0, bool live, float M, float l_half) {
            const int ub = m & 1;
            if (!finish()) return false;
            bool r = pipe_wait<true>(&bars[QB_U_DONE0 + ub], (m >> 1) & 1, sFail, 32);
            if (!r) return false;
            tc_fence_after();
            const uint32_t tU = tl + ub * 256 + 128 + ch * HD;
            float* red = sRed + ub * 8 * (D + 4);
            constexpr int NC = HD / 32;
#pragma unroll
            for (int c = 0; c < NC; ++c) {      // unrolled: rVr must be indexed with constants to stay in registers
                // U is rounded to BF16 pairs and multiplied by the packed Vr words as they are: two instructions a pair,
                // and the lane sums work on BF16 pairs anyway
                uint32_t w[16];
                {
                    uint32_t u[16];
                    tmem_ld16(tU + c * 32, u);
                    tmem_wait_ld();
#pragma unroll
                    for (int t = 0; t < 16; t += 2)
                        w[t >> 1] = mul_bf16x2(pack_bf16x2(__uint_as_float(u[t]), __uint_as_float(u[t + 1])),
                                               rVr[c * 16 + (t >> 1)]);
                }
                {
                    uint32_t u[16];
                    tmem_ld16(tU + c * 32 + 16, u);
                    tmem_wait_ld();
                    if (c == NC - 1) {
                        // U is in registers: a later product may overwrite it
                        tc_fence_before();
                        warp_arrive(&bars[QB_U_FREE0 + ub], lane);
                    }
#pragma unroll
                    for (int t = 0; t < 16; t += 2)
                        w[8 + (t >> 1)] = mul_bf16x2(pack_bf16x2(__uint_as_float(u[t]), __uint_as_float(u[t + 1])),
                                                     rVr[c * 16 + 8 + (t >> 1)]);
                }
                if (W == 16) {
                    float r0, r1;
                    halfwarp_transpose_sum_words(w, lane, r0, r1);
                    red[unit * (D + 4) + ch * HD + c * 32 + 2 * (lane & 15)] = r0;
                    red[unit * (D + 4) + ch * HD + c * 32 + 2 * (lane & 15) + 1] = r1;
                } else {
                    const float s = warp_transpose_sum_words(w, lane);
                    red[unit * (D + 4) + ch * HD + c * 32 + lane] = s;
                }
            }
            {
                float wl = l_half;
#pragma unroll
                for (int o = (W == 16 ? 8 : 16); o >= 1; o >>= 1) wl += __shfl_xor_sync(0xFFFFFFFFu, wl, o);
                if ((lane & (W == 16 ? 15 : 31)) == 0) {
                    red[unit * (D + 4) + D + ch] = wl;
                    if (ch == 0) {
                        red[unit * (D + 4) + D + 2] = M;
                        red[unit * (D + 4) + D + 3] = live ? 1.f : 0.f;
                    }
                }
            }
            warp_arrive(&bars[QB_E_SYNC], lane);
            fin_pending = true; fin_m = m; fin_row = row0; fin_off = off0;
            return true;
        };
        // Tile t takes over: QB keys enter the column ring (forward: the Vs ring rows are this role's to
        // replace, every U product that read the old rows is complete because the caller has drained its
        // epilogues) and this thread's row may change key.
        auto ring_update = [&](int t) {
            const int i0 = q0 + t * QBN;
            if (!pipe_wait<true>(&bars[QB_NEXT_READY0 + ((t - 1) & (KEY_TILES - 1))], ((t - 1) / KEY_TILES) & 1, sFail, 34)) return false;
            if (!DQ && tid < QBN * CH) {
                const int kr = tid / CH, c = tid % CH, key = i0 + kr;
                *reinterpret_cast<uint4*>(sVs + sw128_offset<RING>(key & (RING - 1), c)) =
                    *reinterpret_cast<const uint4*>(key_row(3, key) + c * 16);
            }
            const int knew = ring_key_w<W>(i0 + eg, ejs);
            if (knew != kcur) {
                kcur = knew;
                const uint4* v4 = reinterpret_cast<const uint4*>(key_row(DQ ? 0 : 1, knew) + ch * HD * 2);
#pragma unroll
                for (int c = 0; c < VW / 4; ++c) {
                    const uint4 v = v4[c];
                    rVr[4 * c] = v.x; rVr[4 * c + 1] = v.y; rVr[4 * c + 2] = v.z; rVr[4 * c + 3] = v.w;
                }
            }
            if (!DQ) fence_async_smem();
            return true;
        };
        int n = 0;
        bool ok = true, pend = false, pend_live = false;
        int pend_n = 0;
        size_t pend_row = 0, pend_off = 0;
        float pend_M = 0.f, pend_l = 0.f;
        // dQ mode: the forward statistics and delta of this thread's query for the next head, fetched a head ahead
        float pre_m = 0.f, pre_l = 0.f, pre_d = 0.f;
        auto prefetch = [&](size_t row) {
            if (DQ) { pre_m = __ldg(p.m_in + row); pre_l = __ldg(p.l_in + row); pre_d = __ldg(p.delta + row); }
        };
        prefetch(row_at(q0 + eg, 0));
#pragma unroll 1
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int i0 = q0 + t * QBN, i_last = i0 + QBN - 1;
            // visibility of every query of the tile, of this thread's own query (vw) and of the queries whose
            // rows this warp holds (col_any: the warp-uniform test for skipping a 32-column chunk)
            uint32_t live_vis = 0, vw[4] = {0, 0, 0, 0}, col_any[4] = {0, 0, 0, 0};
#pragma unroll 1
            for (int gg = 0; gg < QBN; ++gg) {
                uint32_t w4[4];
                column_visibility(mask_b.row(i0 + gg), i0 + gg, i_last,
                                  p.window, lane, w4);
                if ((w4[0] | w4[1] | w4[2] | w4[3]) != 0) live_vis |= 1u << gg;
                if (gg == eg) { vw[0] = w4[0]; vw[1] = w4[1]; vw[2] = w4[2]; vw[3] = w4[3]; }
                if (gg * W < (quarter + 1) * 32 && (gg + 1) * W > quarter * 32) {
                    col_any[0] |= w4[0]; col_any[1] |= w4[1]; col_any[2] |= w4[2]; col_any[3] |= w4[3];
                }
            }
            const int n_vis = __popc(vw[0]) + __popc(vw[1]) + __popc(vw[2]) + __popc(vw[3]);
            const bool work = live_vis != 0;
#pragma unroll 1
            for (int hh = 0; hh < G && ok; ++hh) {
                const size_t row0 = row_at(i0, hh);
                const bool boundary = hh == 0 && t > 0;
                const float m_i = pre_m, l_i = pre_l, dlt = pre_d;
                if (DQ) {
                    if (hh + 1 < G) prefetch(row_at(i0 + eg, hh + 1));
                    else if (t + 1 < n_tiles) prefetch(row_at(i0 + QBN + eg, 0));
                }
                if (!work) {
                    if (pend) { ok = epilogue(pend_n, pend_row, pend_off, pend_live, pend_M, pend_l); pend = false; }
                    if (!ok) break;
                    if (boundary) ok = ring_update(t);
                    if (!ok) break;
                    for (int idx = tid; idx < QBN * D; idx += PIPE_E_THREADS) {
                        const size_t row = row0 + idx / D;
                        const size_t at = qoff_at(i0 + idx / D, hh) + idx % D;
                        if (DQ) p.dQ[at] = __float2bfloat16(0.f);
                        else {
                            p.Y[at] = __float2bfloat16(0.f);
                            if (p.Y_act) p.Y_act[at] = __float2bfloat16(0.f);
                            if (idx % D == 0) { p.m[row] = NEG_INF_F; p.l[row] = 0.f; }
                        }
                    }
                    continue;
                }
                // After a boundary's ring_update kcur names this tile's key.  In the forward that update comes
                // before the exponential pass, in the dQ mode after this head's pass: the key's visibility is
                // therefore derived from the row slot, not from kcur.
                const int my_key = ring_key_w<W>(i0 + eg, ejs);
                const bool my_vis = my_key >= 0 && ((vw[(my_key & (RING - 1)) >> 5] >> (my_key & 31)) & 1u);
                const bool live_g = (live_vis >> eg) & 1u;
                const int xb = n & 1;
                const uint32_t tX = tl + xb * 256 + ch * 64;          // this thread's 64 score columns
                ok = pipe_wait<true>(&bars[QB_X_DONE0 + xb], (n >> 1) & 1, sFail, 30);
                if (!ok) break;
                tc_fence_after();
                if (!DQ) {
                    // ---- maximum over this thread's visible columns, then over the rows of its query
                    float mh0 = -INFINITY, mh1 = -INFINITY, mh2 = -INFINITY, mh3 = -INFINITY;
#pragma unroll 1
                    for (int cc = 0; cc < 2; ++cc) {
                        if (col_any[ch * 2 + cc] == 0) continue;          // warp-uniform
                        uint32_t x[32];
                        tmem_ld32(tX + cc * 32, x);
                        tmem_wait_ld();
                        const uint32_t cw = my_vis ? vw[ch * 2 + cc] : 0u;
#pragma unroll
                        for (int t4 = 0; t4 < 32; t4 += 4) {
                            if ((cw >> t4) & 1u) mh0 = fmaxf(mh0, __uint_as_float(x[t4]));
                            if ((cw >> (t4 + 1)) & 1u) mh1 = fmaxf(mh1, __uint_as_float(x[t4 + 1]));
                            if ((cw >> (t4 + 2)) & 1u) mh2 = fmaxf(mh2, __uint_as_float(x[t4 + 2]));
                            if ((cw >> (t4 + 3)) & 1u) mh3 = fmaxf(mh3, __uint_as_float(x[t4 + 3]));
                        }
                    }
                    {
                        float m_w = fmaxf(fmaxf(mh0, mh1), fmaxf(mh2, mh3));
#pragma unroll
                        for (int o = (W == 16 ? 8 : 16); o >= 1; o >>= 1) m_w = fmaxf(m_w, __shfl_xor_sync(0xFFFFFFFFu, m_w, o));
                        if ((lane & 15) == 0) sMpart[xb * 16 + warp * 2 + (lane >> 4)] = m_w;
                    }
                    warp_arrive(&bars[QB_M_SYNC], lane);
                    // ---- epilogue of the previous head, behind its U product; then the rows of the entering keys
                    if (pend) { ok = epilogue(pend_n, pend_row, pend_off, pend_live, pend_M, pend_l); pend = false; }
                    if (ok && boundary) ok = ring_update(t);
                    if (!ok) break;
                    ok = pipe_wait<true>(&bars[QB_M_SYNC], n & 1, sFail, 31);
                    if (!ok) break;
                    const float* mp = sMpart + xb * 16;
                    float M = -INFINITY;
#pragma unroll
                    for (int e = 0; e < 16; ++e)                       // half-warp entries of this thread's row group
                        if ((((e >> 1) & 3) * 32 + (e & 1) * 16) / W == eg) M = fmaxf(M, mp[e]);
                    if (!live_g) M = 0.f;
                    const float mc = M * c2;
                    // ---- P = exp2((x - M) c2), BF16 over the first 32 of this thread's columns; half-row sum
                    const uint64_t c2p = pair_f32(c2, c2), mcp = pair_f32(-mc, -mc);     // packed FP32: two columns an instruction
                    uint64_t ls0 = pair_f32(0.f, 0.f), ls1 = ls0;
#pragma unroll 1
                    for (int cc = 0; cc < 2; ++cc) {
                        uint32_t pk[16];
                        if (col_any[ch * 2 + cc] == 0) {
#pragma unroll
                            for (int t4 = 0; t4 < 16; ++t4) pk[t4] = 0u;
                        } else {
                            uint32_t x[32];
                            tmem_ld32(tX + cc * 32, x);
                            tmem_wait_ld();
                            const uint32_t cw = my_vis ? vw[ch * 2 + cc] : 0u;
#pragma unroll
                            for (int t4 = 0; t4 < 32; t4 += 2) {
                                float a0, a1;
                                unpair_f32(fma_f32x2(pair_b32(x[t4], x[t4 + 1]), c2p, mcp), a0, a1);
                                float e0 = fast_exp2(a0), e1 = fast_exp2(a1);
                                if (!((cw >> t4) & 1u)) e0 = 0.f;
                                if (!((cw >> (t4 + 1)) & 1u)) e1 = 0.f;
                                if (t4 & 2) ls1 = add_f32x2(ls1, pair_f32(e0, e1));
                                else ls0 = add_f32x2(ls0, pair_f32(e0, e1));
                                pk[t4 >> 1] = pack_bf16x2(e0, e1);
                            }
                        }
                        tmem_st16(tX + cc * 16, pk);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    // P_full also tells the MMA warp that the Vs ring rows are current (ring_update above)
                    warp_arrive(&bars[QB_P_FULL0 + xb], lane);
                    pend = true; pend_n = n; pend_row = row0; pend_off = qoff_at(i0, hh); pend_live = live_g; pend_M = M;
                    {
                        float s0, s1;
                        unpair_f32(add_f32x2(ls0, ls1), s0, s1);
                        pend_l = s0 + s1;
                    }
                } else {
                    // ---- gA = P o (dP - delta), P = exp2(x c2 - lse) from the forward's statistics; BF16 over the
                    //      first 32 of this thread's score columns.  A query with one visible key gets exact zeros.
                    const bool live_q = live_g && l_i > 0.f;
                    const float lse2 = live_q ? m_i * LOG2E + __log2f(l_i) : 0.f;
                    const bool zero_all = !live_q || n_vis == 1 || !my_vis;
                    const uint64_t c2p = pair_f32(c2, c2), lsep = pair_f32(-lse2, -lse2), dltp = pair_f32(-dlt, -dlt);
#pragma unroll 1
                    for (int cc = 0; cc < 2; ++cc) {
                        uint32_t pk[16];
                        if (col_any[ch * 2 + cc] == 0) {
#pragma unroll
                            for (int t4 = 0; t4 < 16; ++t4) pk[t4] = 0u;
                        } else {
                            const uint32_t cw = zero_all ? 0u : vw[ch * 2 + cc];
#pragma unroll
                            for (int r16 = 0; r16 < 2; ++r16) {
                                uint32_t x[16], dp[16];
                                tmem_ld16(tX + cc * 32 + r16 * 16, x);
                                tmem_ld16(tX + 128 + cc * 32 + r16 * 16, dp);
                                tmem_wait_ld();
#pragma unroll
                                for (int t4 = 0; t4 < 16; t4 += 2) {
                                    float a0, a1, d0, d1;
                                    unpair_f32(fma_f32x2(pair_b32(x[t4], x[t4 + 1]), c2p, lsep), a0, a1);
                                    unpair_f32(add_f32x2(pair_b32(dp[t4], dp[t4 + 1]), dltp), d0, d1);
                                    float g0 = fast_exp2(a0) * d0, g1 = fast_exp2(a1) * d1;
                                    if (!((cw >> (r16 * 16 + t4)) & 1u)) g0 = 0.f;
                                    if (!((cw >> (r16 * 16 + t4 + 1)) & 1u)) g1 = 0.f;
                                    pk[r16 * 8 + (t4 >> 1)] = pack_bf16x2(g0, g1);
                                }
                            }
                        }
                        tmem_st16(tX + cc * 16, pk);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    warp_arrive(&bars[QB_P_FULL0 + xb], lane);
                    // ---- collapse of the previous head's Ug, then this tile's row registers
                    if (pend) { ok = epilogue(pend_n, pend_row, pend_off, pend_live, pend_M, pend_l); pend = false; }
                    if (ok && boundary) ok = ring_update(t);
                    if (!ok) break;
                    pend = true; pend_n = n; pend_row = row0; pend_off = qoff_at(i0, hh); pend_live = live_q; pend_M = 0.f; pend_l = 0.f;
                }
                ++n;
            }
        }
        if (ok && pend) ok = epilogue(pend_n, pend_row, pend_off, pend_live, pend_M, pend_l);
        if (ok) ok = finish();
    }
    tc_fence_before();
    __syncthreads();
    if (*sFail && tid == 0) atomicExch(p.status, 200 + *sFail);
    if (is_mma) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace sgpack
