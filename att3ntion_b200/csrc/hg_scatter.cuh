// Scatter outputs of the three-gather operator and their gradients, on CUDA cores.
//
// With x[i,j,k] = scale * sum_d Q_i[d] R_j[d] S_k[d] and the three anchored softmaxes Aq (over (j,k)
// for fixed i), Ar (over (i,k) for fixed j), As (over (i,j) for fixed k), the scatter outputs weight
// each cell with the product of the two softmaxes that are NOT anchored at the output index
// (cpp/torch_reference.cpp:51-54, cuda/forward.cu:941-1249):
//
//   Y_q_[i] = sum_{j,k} Ar As  Vr2[j] o Vs2[k]      Y_r_[j] = sum_{i,k} Aq As  Vq2[i] o Vs2[k]
//   Y_s_[k] = sum_{i,j} Aq Ar  Vq2[i] o Vr2[j]
//
// All three are one generic form with roles (a, u, v): output index a, the two other indices u, v,
//   out[a] = sum_{u,v} W[a,u,v]  Vu2[u] o Vv2[v],    W = Pu Pv,   Pu = exp(x - m_u[u]) / l_u[u]
// where (m_u, l_u) are the statistics of the softmax anchored at u (taken over (a, v)), likewise Pv.
// Both exponents are <= 0 because each maximum is taken over a set that contains the cell.
//
// Gradients of one such term under the cotangent g[a] (c = sum_d g[a,d] Vu2[u,d] Vv2[v,d]):
//   dVu2[u] = sum_{a,v} W  g[a] o Vv2[v]            (dVv2 by exchanging u and v)
//   dx      = 2 W c - Pu Cu[u] - Pv Cv[v],   Cu[u] = sum_{a,v} W c = Vu2[u] . dVu2[u],  Cv likewise
//   dA[a]   = scale sum_{u,v} dx  U_u o V_v ,  dU[u] = scale sum_{a,v} dx  A_a o V_v   (dV by exchange)
// (the reference's scalar kernels compute the same sums: cuda/backward.cu:175-316, 949-1613).
//
// This is the operator's fallback path in the reference as well (scalar kernels, used only when a
// second value tensor is non-zero); it is written for correctness and moderate speed: one thread per
// (a, u) pair walks v, scores are recomputed from shared-memory rows, sums over u stay in the warp,
// sums over a go through shared-memory atomics, and the FP32 result planes are updated with global
// atomics (so, unlike the gather kernels, repeated calls may differ in the last bit).
#pragma once

#include <cuda_bf16.h>
#include <cstdint>

namespace hgscatter {

constexpr int T = 16;              // tile edge: 16 x 16 (a, u) pairs per CTA, 16 v per step
constexpr int THREADS = T * T;

struct Params {
    const __nv_bfloat16* A;        // keys of the output index        [B,H,N,D]
    const __nv_bfloat16* U;        // keys of the first other index
    const __nv_bfloat16* V;        // keys of the second other index
    const __nv_bfloat16* Vu2;      // second value tensor of u
    const __nv_bfloat16* Vv2;      // second value tensor of v
    const __nv_bfloat16* G;        // cotangent of out (modes 1, 2)
    const float* m_u; const float* l_u;    // statistics of the softmax anchored at u   [B,H,N]
    const float* m_v; const float* l_v;
    const float* Cu; const float* Cv;      // mode 2: correction sums                  [B,H,N]
    const uint8_t* mask;           // [B,N,N] (anchor, other) or null
    __nv_bfloat16* out_bf16;       // mode 0: the scatter output                        [B,H,N,D]
    float* out_a;                  // mode 2: dA plane                                  [B,H,N,D] FP32
    float* out_u;                  // mode 1: dVu2 plane; mode 2: dU plane
    int B, H, N, D, n_valid;
    float scale;
};

__device__ __forceinline__ float bf(const __nv_bfloat16 v) { return __bfloat162float(v); }

// MODE 0: out[a] = sum_u Vu2[u] o t,  t = sum_v W Vv2[v]         (forward; the CTA walks every u tile
//         itself, so the output needs no atomics and no FP32 staging)
// MODE 1: out_u[u] += g[a]  o t                                   (gradient of Vu2)
// MODE 2: s = sum_v dx V_v;  out_a[a] += scale U_u o s,  out_u[u] += scale A_a o s   (key gradients)
// DH = columns of the D-vector kept per thread; blockIdx.z also enumerates the D / DH column blocks.
template <int D, int DH, int MODE>
__global__ void __launch_bounds__(THREADS, 1) hg_scatter_kernel(const Params p) {
    extern __shared__ float sm[];
    float* sA = sm;                    // [T][D]
    float* sU = sA + T * D;            // [T][D]
    float* sV = sU + T * D;            // [T][D]
    float* sVv = sV + T * D;           // [T][DH]   Vv2 rows (modes 0, 1) or V rows' column block (mode 2 reuses sV)
    float* sG = sVv + T * DH;          // [T][D]    mode 2: g[a] rows;  mode 1: g[a] column block in the first T*DH
    float* sW2 = sG + T * D;           // [T][D]    mode 2: Vu2[u] rows
    float* sVv2full = sW2 + T * D;     // [T][D]    mode 2: Vv2[v] rows
    float* sOutU = sVv2full + T * D;   // [T][DH]   sums over a
    __shared__ float s_mv[T], s_lv[T], s_cv[T];
    __shared__ uint8_t s_mask_va[T][T], s_mask_vu[T][T];     // mask[v][a], mask[v][u]

    constexpr int NH = D / DH;
    const int tid = threadIdx.x;
    const int ta = tid / T, tu = tid % T;
    const int bh = blockIdx.z / NH, dblk = blockIdx.z % NH;
    const int b = bh / p.H;
    const int a0 = blockIdx.x * T;
    const int a = a0 + ta;
    const int N = p.N;
    const int n_keys = (p.n_valid > 0 && p.n_valid < N) ? p.n_valid : N;
    const size_t base = static_cast<size_t>(bh) * N;
    const uint8_t* mask_b = p.mask ? p.mask + static_cast<size_t>(b) * N * N : nullptr;

    float acc[MODE == 0 ? DH : 1];
#pragma unroll
    for (int d = 0; d < (MODE == 0 ? DH : 1); ++d) acc[d] = 0.f;
    const int u_first = MODE == 0 ? 0 : blockIdx.y * T, u_last = MODE == 0 ? N : u_first + T;
    for (int u0 = u_first; u0 < u_last; u0 += T) {
    const int u = u0 + tu;
    __syncthreads();
    // rows of the CTA's a and u tiles
    for (int idx = tid; idx < T * D; idx += THREADS) {
        const int r = idx / D, d = idx % D;
        sA[idx] = bf(p.A[(base + a0 + r) * D + d]);
        sU[idx] = bf(p.U[(base + u0 + r) * D + d]);
        if (MODE == 2) {
            sG[idx] = bf(p.G[(base + a0 + r) * D + d]);
            sW2[idx] = bf(p.Vu2[(base + u0 + r) * D + d]);
        }
    }
    for (int idx = tid; idx < T * DH; idx += THREADS) {
        sOutU[idx] = 0.f;
        if (MODE == 1) {
            const int r = idx / DH, d = idx % DH;
            sG[idx] = bf(p.G[(base + a0 + r) * D + dblk * DH + d]);
        }
    }
    const float mu = p.m_u[base + u], lu = p.l_u[base + u];
    const float inv_lu = lu > 0.f ? 1.f / lu : 0.f;
    const float cu = MODE == 2 ? p.Cu[base + u] : 0.f;
    const bool in_range = a < n_keys && u < n_keys;
    // an anchor without any visible cell has l = 0 (and m = -1e30): its softmax is identically zero
    const bool u_sees_a = in_range && lu > 0.f && (!mask_b || mask_b[static_cast<size_t>(u) * N + a] != 0);

    float t[DH];
#pragma unroll
    for (int d = 0; d < DH; ++d) t[d] = 0.f;

    for (int v0 = 0; v0 < N; v0 += T) {
        __syncthreads();
        for (int idx = tid; idx < T * D; idx += THREADS) {
            const int r = idx / D, d = idx % D;
            sV[idx] = bf(p.V[(base + v0 + r) * D + d]);
            if (MODE == 2) sVv2full[idx] = bf(p.Vv2[(base + v0 + r) * D + d]);
        }
        if (MODE != 2)
            for (int idx = tid; idx < T * DH; idx += THREADS) {
                const int r = idx / DH, d = idx % DH;
                sVv[idx] = bf(p.Vv2[(base + v0 + r) * D + dblk * DH + d]);
            }
        if (tid < T) {
            s_mv[tid] = p.m_v[base + v0 + tid];
            const float lv = p.l_v[base + v0 + tid];
            s_lv[tid] = lv > 0.f ? 1.f / lv : 0.f;
            s_cv[tid] = MODE == 2 ? p.Cv[base + v0 + tid] : 0.f;
        }
        {   // mask[v][a] and mask[v][u] for the tile (anchor v sees a, u)
            const int r = tid / T, c = tid % T;
            const int v = v0 + r;
            const bool vin = v < n_keys;
            s_mask_va[r][c] = vin && (!mask_b || mask_b[static_cast<size_t>(v) * N + a0 + c] != 0);
            s_mask_vu[r][c] = vin && (!mask_b || mask_b[static_cast<size_t>(v) * N + u0 + c] != 0);
        }
        __syncthreads();

        // scores (and, for the key gradients, c = sum_d g[a] Vu2[u] Vv2[v]) of this thread's 16 cells
        float x[T], cc[T];
#pragma unroll
        for (int k = 0; k < T; ++k) { x[k] = 0.f; cc[k] = 0.f; }
        for (int d = 0; d < D; d += 4) {
            const float4 qa = *reinterpret_cast<const float4*>(sA + ta * D + d);
            const float4 qu = *reinterpret_cast<const float4*>(sU + tu * D + d);
            const float4 qr = make_float4(qa.x * qu.x, qa.y * qu.y, qa.z * qu.z, qa.w * qu.w);
            float4 gw = make_float4(0.f, 0.f, 0.f, 0.f);
            if (MODE == 2) {
                const float4 g4 = *reinterpret_cast<const float4*>(sG + ta * D + d);
                const float4 w4 = *reinterpret_cast<const float4*>(sW2 + tu * D + d);
                gw = make_float4(g4.x * w4.x, g4.y * w4.y, g4.z * w4.z, g4.w * w4.w);
            }
#pragma unroll
            for (int k = 0; k < T; ++k) {
                const float4 sv = *reinterpret_cast<const float4*>(sV + k * D + d);
                x[k] += qr.x * sv.x + qr.y * sv.y + qr.z * sv.z + qr.w * sv.w;
                if (MODE == 2) {
                    const float4 vv = *reinterpret_cast<const float4*>(sVv2full + k * D + d);
                    cc[k] += gw.x * vv.x + gw.y * vv.y + gw.z * vv.z + gw.w * vv.w;
                }
            }
        }
        // weights of the 16 cells
        float w[T];
#pragma unroll
        for (int k = 0; k < T; ++k) {
            const int v = v0 + k;
            // Pu is live iff anchor u sees a and v; Pv iff anchor v sees a and u (each softmax has its own
            // support, and the correction terms of the gradient follow the support of their own factor)
            const bool live_u = u_sees_a && v < n_keys && (!mask_b || mask_b[static_cast<size_t>(u) * N + v] != 0);
            const bool live_v = in_range && s_lv[k] > 0.f && s_mask_va[k][ta] && s_mask_vu[k][tu];
            const float xs = x[k] * p.scale;
            const float pu = live_u ? __expf(xs - mu) * inv_lu : 0.f;
            const float pv = live_v ? __expf(xs - s_mv[k]) * s_lv[k] : 0.f;
            if (MODE == 2) w[k] = 2.f * pu * pv * cc[k] - pu * cu - pv * s_cv[k];
            else w[k] = pu * pv;
        }
        // t += sum_k w[k] * row_k, row = Vv2 (modes 0, 1) or V (mode 2), column block dblk
#pragma unroll
        for (int k = 0; k < T; ++k) {
            const float wk = w[k];
            const float* row = MODE == 2 ? sV + k * D + dblk * DH : sVv + k * DH;
#pragma unroll
            for (int d = 0; d < DH; d += 4) {
                const float4 r4 = *reinterpret_cast<const float4*>(row + d);
                t[d] += wk * r4.x; t[d + 1] += wk * r4.y; t[d + 2] += wk * r4.z; t[d + 3] += wk * r4.w;
            }
        }
    }
    __syncthreads();

    if (MODE == 0) {
        // this u tile's share of out[a]; t starts over for the next tile
        const __nv_bfloat16* urow = p.Vu2 + (base + u) * D + dblk * DH;
#pragma unroll
        for (int d = 0; d < DH; ++d) {
            acc[d] += bf(urow[d]) * t[d];
            t[d] = 0.f;
        }
    }
    // ---- output index a (mode 2): multiply by the u row, sum over the 16 u of the half warp
    if (MODE == 2 && p.out_a) {      // null: the caller already has this term (second launch with u, v exchanged)
        const __nv_bfloat16* urow = p.U + (base + u) * D + dblk * DH;
#pragma unroll
        for (int d = 0; d < DH; ++d) {
            float val = p.scale * bf(urow[d]) * t[d];
#pragma unroll
            for (int o = 8; o >= 1; o >>= 1) val += __shfl_xor_sync(0xFFFFFFFFu, val, o);
            if (tu == 0) atomicAdd(p.out_a + (base + a) * D + dblk * DH + d, val);
        }
    }
    // ---- output index u (modes 1, 2): multiply by the a row, sum over the 16 a of the CTA
    if (MODE == 1 || MODE == 2) {
        const float mul = MODE == 2 ? p.scale : 1.f;
#pragma unroll
        for (int d = 0; d < DH; ++d) {
            const float arow = MODE == 1 ? sG[ta * DH + d] : sA[ta * D + dblk * DH + d];
            float val = mul * arow * t[d];
            val += __shfl_xor_sync(0xFFFFFFFFu, val, 16);          // the two a of this warp
            if ((tid & 16) == 0) atomicAdd(sOutU + tu * DH + d, val);
        }
        __syncthreads();
        for (int idx = tid; idx < T * DH; idx += THREADS) {
            const int r = idx / DH, d = idx % DH;
            atomicAdd(p.out_u + (base + u0 + r) * D + dblk * DH + d, sOutU[idx]);
        }
    }
    }   // u tiles
    if (MODE == 0) {
#pragma unroll
        for (int d = 0; d < DH; ++d) {
            float val = acc[d];
#pragma unroll
            for (int o = 8; o >= 1; o >>= 1) val += __shfl_xor_sync(0xFFFFFFFFu, val, o);
            if (tu == 0) p.out_bf16[(base + a) * D + dblk * DH + d] = __float2bfloat16(val);
        }
    }
}

template <int D, int DH>
constexpr size_t smem_bytes() { return sizeof(float) * (T * D * 6 + T * DH * 2); }

// row . row over D for two [n, D] tensors (bf16 x fp32): C[n] = sum_d V2[n,d] * dV2[n,d]
__global__ void rowdot_kernel(const __nv_bfloat16* v2, const float* dv2, float* out, size_t rows, int D) {
    const size_t warp = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) / 32;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    float s = 0.f;
    for (int d = lane; d < D; d += 32) s += __bfloat162float(v2[warp * D + d]) * dv2[warp * D + d];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if (lane == 0) out[warp] = s;
}

}  // namespace hgscatter
