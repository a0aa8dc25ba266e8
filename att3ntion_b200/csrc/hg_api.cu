// Dense anchored-gather launchers and the C-ABI entry points of the three-gather
// hypergraph attention, which is three anchored gathers with permuted roles
// (forward) and the sum of their gradients (backward).
#include <algorithm>
#include <cmath>

#include "att3_abi_internal.h"
#include "ag_dense_bwd.cuh"
#include "hg_scatter.cuh"

namespace {

__device__ int g_ag_status = 0;

int* ag_status_ptr() {
    int* p = nullptr;
    cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ag_status);
    return p;
}

template <typename K>
int opt_in_smem(K kernel, int bytes, const char* who) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    return e == cudaSuccess ? ATT3_OK : att3::set_cuda_error(e, who);
}

template <int DP>
int launch_fwd(const agdense::FwdParams& p, cudaStream_t st) {
    using L = agdense::FwdSmem<DP>;
    if (int rc = opt_in_smem(agdense::ag_dense_fwd_kernel<DP>, L::ALLOC, "dense gather forward: shared-memory opt-in")) return rc;
    dim3 grid((p.N + p.group - 1) / p.group, p.H, p.B);
    att3::TimedLaunch timed(att3::K_DENSE_FWD, st);
    agdense::ag_dense_fwd_kernel<DP><<<grid, agdense::NTHREADS, L::ALLOC, st>>>(p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ATT3_OK : att3::set_cuda_error(e, "dense gather forward: launch");
}

template <int DP, bool WITH_DA>
int launch_bwd(const agdense::BwdParams& p, int n_tiles, cudaStream_t st) {
    using L = agdense::BwdSmem<DP, WITH_DA>;
    if (int rc = opt_in_smem(agdense::ag_dense_bwd_kernel<DP, WITH_DA>, L::ALLOC, "dense gather backward: shared-memory opt-in"))
        return rc;
    dim3 grid(n_tiles * p.a_chunks, p.H, p.B);
    att3::TimedLaunch timed(att3::K_DENSE_BWD, st);
    agdense::ag_dense_bwd_kernel<DP, WITH_DA><<<grid, agdense::BWD_THREADS, L::ALLOC, st>>>(p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ATT3_OK : att3::set_cuda_error(e, "dense gather backward: launch");
}

int grid_for(size_t n) { return static_cast<int>(std::min<size_t>((n + 255) / 256, 148 * 8)); }

}  // namespace

namespace att3 {

int dense_status_read_and_clear(int* out) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_ag_status, sizeof(int));
    if (e != cudaSuccess) return set_cuda_error(e, "att3_device_status: read");
    if (*out) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_ag_status, &zero, sizeof(int));
    }
    return ATT3_OK;
}

int dense_tiles(int N, int n_valid) {
    const int n_keys = (n_valid > 0 && n_valid < N) ? n_valid : N;
    return (n_keys + agdense::TILE - 1) / agdense::TILE;
}

int dense_gather_forward(const void* A, const void* Rw, const void* C, const void* Vrow, const void* Vcol,
                         const uint8_t* mask, void* Y, float* m, float* l, int B, int H, int N, int D, int n_valid,
                         cudaStream_t st) {
    agdense::FwdParams p;
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.Rw = static_cast<const __nv_bfloat16*>(Rw);
    p.C = static_cast<const __nv_bfloat16*>(C);
    p.Vrow = static_cast<const __nv_bfloat16*>(Vrow);
    p.Vcol = static_cast<const __nv_bfloat16*>(Vcol);
    p.mask = mask;
    p.Y = static_cast<__nv_bfloat16*>(Y);
    p.m = m; p.l = l;
    p.B = B; p.H = H; p.N = N; p.D = D; p.n_valid = n_valid;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = ag_status_ptr();
    // anchors per CTA: enough CTAs to fill the device twice over, at most 16 anchors each
    const long ctas_at_16 = static_cast<long>((N + 15) / 16) * H * B;
    p.group = ctas_at_16 >= 2L * sm_count() ? 16 : (ctas_at_16 * 2 >= 2L * sm_count() ? 8 : 4);
    return D > 64 ? launch_fwd<128>(p, st) : launch_fwd<64>(p, st);
}

int dense_gather_backward_side(const void* A, const void* dY, const void* Y, const float* m, const float* l,
                               const void* Ka, const void* Va, const void* Kb, const void* Vb, const uint8_t* mask,
                               float* dKb, float* dVb, float* dA_part, int B, int H, int N, int D, int n_valid,
                               cudaStream_t st, float* chunk_scratch) {
    agdense::BwdParams p;
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.dY = static_cast<const __nv_bfloat16*>(dY);
    p.Y = static_cast<const __nv_bfloat16*>(Y);
    p.m = m; p.l = l;
    p.Ka = static_cast<const __nv_bfloat16*>(Ka);
    p.Va = static_cast<const __nv_bfloat16*>(Va);
    p.Kb = static_cast<const __nv_bfloat16*>(Kb);
    p.Vb = static_cast<const __nv_bfloat16*>(Vb);
    p.mask = mask;
    p.dKb = dKb; p.dVb = dVb; p.dA_part = dA_part;
    p.B = B; p.H = H; p.N = N; p.D = D; p.n_valid = n_valid;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = ag_status_ptr();
    const int nt = dense_tiles(N, n_valid);
    // One CTA per (own tile, batch, head) leaves most SMs idle for short sequences: split the anchors in two
    // when that still fits the machine and the caller has given room for the second chunk's planes.
    const size_t plane = static_cast<size_t>(B) * H * N * D;
    p.a_chunks = (chunk_scratch && 2 * nt * B * H <= sm_count() && N >= 2) ? 2 : 1;
    p.dKb1 = chunk_scratch;
    p.dVb1 = chunk_scratch ? chunk_scratch + plane : nullptr;
    if (p.a_chunks == 2) cudaMemsetAsync(chunk_scratch, 0, 2 * plane * sizeof(float), st);
    int rc;
    if (dA_part) rc = D > 64 ? launch_bwd<128, true>(p, nt, st) : launch_bwd<64, true>(p, nt, st);
    else rc = D > 64 ? launch_bwd<128, false>(p, nt, st) : launch_bwd<64, false>(p, nt, st);
    if (rc || p.a_chunks == 1) return rc;
    if ((rc = add_planes(p.dKb1, 1, plane, dKb, st))) return rc;
    return add_planes(p.dVb1, 1, plane, dVb, st);
}

int add_planes(const float* src, int n_src, size_t plane, float* acc, cudaStream_t st) {
    TimedLaunch timed(K_HG_AUX, st);
    agdense::ag_add_planes<<<grid_for(plane), 256, 0, st>>>(src, n_src, plane, acc, plane);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ATT3_OK : set_cuda_error(e, "add_planes: launch");
}

int plane_to_bf16(const float* src, void* out, size_t n, cudaStream_t st) {
    TimedLaunch timed(K_HG_AUX, st);
    agdense::ag_sum_planes_to_bf16<<<grid_for(n), 256, 0, st>>>(src, 1, n, static_cast<__nv_bfloat16*>(out), n);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ATT3_OK : set_cuda_error(e, "plane_to_bf16: launch");
}

}  // namespace att3

// ---------------------------------------------------------------------------------------------
// Scatter terms (CUDA-core kernels, hg_scatter.cuh)
// ---------------------------------------------------------------------------------------------

template <int D, int DH, int MODE>
static int launch_scatter_t(const hgscatter::Params& p, cudaStream_t st) {
    const size_t smem = hgscatter::smem_bytes<D, DH>();
    cudaError_t e = cudaFuncSetAttribute(hgscatter::hg_scatter_kernel<D, DH, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return att3::set_cuda_error(e, "scatter: shared-memory opt-in");
    dim3 grid(p.N / hgscatter::T, MODE == 0 ? 1 : p.N / hgscatter::T, p.B * p.H * (D / DH));
    att3::TimedLaunch timed(att3::K_HG_AUX, st);
    hgscatter::hg_scatter_kernel<D, DH, MODE><<<grid, hgscatter::THREADS, smem, st>>>(p);
    e = cudaGetLastError();
    return e == cudaSuccess ? ATT3_OK : att3::set_cuda_error(e, "scatter: launch");
}

template <int MODE>
static int launch_scatter(const hgscatter::Params& p, cudaStream_t st) {
    switch (p.D) {
        case 16: return launch_scatter_t<16, 16, MODE>(p, st);
        case 32: return launch_scatter_t<32, 32, MODE>(p, st);
        case 64: return launch_scatter_t<64, 64, MODE>(p, st);
        default: return launch_scatter_t<128, 64, MODE>(p, st);
    }
}

// One index of the operator in a given role: its keys, second value tensor and the statistics of the
// softmax anchored at it.
struct ScatterSide {
    const void* keys; const void* v2; const float* m; const float* l;
};

static hgscatter::Params scatter_params(const ScatterSide& a, const ScatterSide& u, const ScatterSide& v,
                                        const uint8_t* mask, int B, int H, int N, int D, int n_valid) {
    hgscatter::Params p{};
    p.A = static_cast<const __nv_bfloat16*>(a.keys);
    p.U = static_cast<const __nv_bfloat16*>(u.keys);
    p.V = static_cast<const __nv_bfloat16*>(v.keys);
    p.Vu2 = static_cast<const __nv_bfloat16*>(u.v2);
    p.Vv2 = static_cast<const __nv_bfloat16*>(v.v2);
    p.m_u = u.m; p.l_u = u.l; p.m_v = v.m; p.l_v = v.l;
    p.mask = mask;
    p.B = B; p.H = H; p.N = N; p.D = D; p.n_valid = n_valid;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    return p;
}

// out[a] = sum_{u,v} Pu Pv Vu2[u] o Vv2[v]   (forward of one scatter output)
static int scatter_forward(const ScatterSide& a, const ScatterSide& u, const ScatterSide& v, const uint8_t* mask,
                           void* out, int B, int H, int N, int D, int n_valid, cudaStream_t st) {
    hgscatter::Params p = scatter_params(a, u, v, mask, B, H, N, D, n_valid);
    p.out_bf16 = static_cast<__nv_bfloat16*>(out);
    return launch_scatter<0>(p, st);
}

// Gradients of one scatter output under the cotangent g: into the FP32 planes of the three key tensors and
// of the two second value tensors.  tmp: two planes + two [B,H,N] vectors of scratch.
static int scatter_backward(const ScatterSide& a, const ScatterSide& u, const ScatterSide& v, const void* g,
                            const uint8_t* mask, float* gA, float* gU, float* gV, float* gVu2, float* gVv2,
                            float* tmp, int B, int H, int N, int D, int n_valid, cudaStream_t st) {
    const size_t plane = static_cast<size_t>(B) * H * N * D, rows = static_cast<size_t>(B) * H * N;
    float *tmpU = tmp, *tmpV = tmp + plane, *Cu = tmp + 2 * plane, *Cv = Cu + rows;
    cudaMemsetAsync(tmp, 0, 2 * plane * sizeof(float), st);
    int rc;
    {   // value gradients of this term alone (their row dots are the softmax corrections)
        hgscatter::Params p = scatter_params(a, u, v, mask, B, H, N, D, n_valid);
        p.G = static_cast<const __nv_bfloat16*>(g);
        p.out_u = tmpU;
        if ((rc = launch_scatter<1>(p, st))) return rc;
        hgscatter::Params q = scatter_params(a, v, u, mask, B, H, N, D, n_valid);
        q.G = p.G;
        q.out_u = tmpV;
        if ((rc = launch_scatter<1>(q, st))) return rc;
    }
    const int wpb = 8;    // warps per block of the row-dot kernel
    const unsigned nblk = static_cast<unsigned>((rows + wpb - 1) / wpb);
    hgscatter::rowdot_kernel<<<nblk, wpb * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(u.v2), tmpU, Cu, rows, D);
    hgscatter::rowdot_kernel<<<nblk, wpb * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(v.v2), tmpV, Cv, rows, D);
    if ((rc = att3::add_planes(tmpU, 1, plane, gVu2, st))) return rc;
    if ((rc = att3::add_planes(tmpV, 1, plane, gVv2, st))) return rc;
    {   // key gradients: (a, u) from the first launch, v from the launch with u and v exchanged
        hgscatter::Params p = scatter_params(a, u, v, mask, B, H, N, D, n_valid);
        p.G = static_cast<const __nv_bfloat16*>(g);
        p.Cu = Cu; p.Cv = Cv;
        p.out_a = gA; p.out_u = gU;
        if ((rc = launch_scatter<2>(p, st))) return rc;
        hgscatter::Params q = scatter_params(a, v, u, mask, B, H, N, D, n_valid);
        q.G = p.G;
        q.Cu = Cv; q.Cv = Cu;
        q.out_a = nullptr; q.out_u = gV;
        if ((rc = launch_scatter<2>(q, st))) return rc;
    }
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ATT3_OK : att3::set_cuda_error(e, "scatter backward: launch");
}

// ---------------------------------------------------------------------------------------------
// Three-gather forward
// ---------------------------------------------------------------------------------------------

static __global__ void fill_stats_kernel(float* m, float* l, size_t n, float mv, float lv) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        m[i] = mv;
        l[i] = lv;
    }
}

static int check_hg(const char* who, int B, int H, int N, int D) {
    if (B <= 0 || H <= 0 || N <= 0) return att3::set_error(ATT3_ERR_INVALID, "%s: empty batch/head/sequence", who);
    if (D != 16 && D != 32 && D != 64 && D != 128)
        return att3::set_error(ATT3_ERR_INVALID, "%s: head dim must be 16, 32, 64 or 128, got %d", who, D);
    if (N % 16 != 0) return att3::set_error(ATT3_ERR_INVALID, "%s: N must be a multiple of 16, got %d", who, N);
    return ATT3_OK;
}

extern "C" int att3_hg_forward(const void* Q, const void* R, const void* S, const void* Vq1, const void* Vq2,
                               const void* Vr1, const void* Vr2, const void* Vs1, const void* Vs2,
                               const uint8_t* mask, void* Yq, void* Yr, void* Ys, void* Yq_, void* Yr_, void* Ys_,
                               float* m_i, float* l_i, float* m_j, float* l_j, float* m_k, float* l_k, int B, int H,
                               int N, int D, int n_valid, int gather_mode, int scatter, void* stream) {
    if (int rc = check_hg("att3_hg_forward", B, H, N, D)) return rc;
    if (!Q || !R || !S || !Vq1 || !Vr1 || !Vs1 || !Yq || !Yr || !Ys || !Yq_ || !Yr_ || !Ys_ || !m_i || !l_i || !m_j ||
        !l_j || !m_k || !l_k)
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_forward: null tensor pointer");
    if (gather_mode != 0 && gather_mode != 1)
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_forward: gather_mode must be 0 or 1, got %d", gather_mode);
    if (scatter && gather_mode != 0)
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_forward: scatter needs all three gathers (gather_mode 0)");
    if (scatter && (!Vq2 || !Vr2 || !Vs2))
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_forward: scatter needs the second value tensors");
    if (!att3::require_sm100("att3_hg_forward")) return ATT3_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t n = static_cast<size_t>(B) * H * N;
    const size_t bytes = n * D * 2;
    // outputs of skipped gathers / scatters read as zero (cuda/forward.cu:1308-1321)
    cudaMemsetAsync(Yq_, 0, bytes, st);
    cudaMemsetAsync(Yr_, 0, bytes, st);
    cudaMemsetAsync(Ys_, 0, bytes, st);
    int rc = att3::dense_gather_forward(Q, R, S, Vr1, Vs1, mask, Yq, m_i, l_i, B, H, N, D, n_valid, st);
    if (rc) return rc;
    att3::count_launch(2);
    if (gather_mode == 1) {
        cudaMemsetAsync(Yr, 0, bytes, st);
        cudaMemsetAsync(Ys, 0, bytes, st);
        // statistics that make the other two softmax weights vanish (cuda/forward.cu:1455-1459)
        fill_stats_kernel<<<148, 256, 0, st>>>(m_j, l_j, n, 1e30f, 1.0f);
        fill_stats_kernel<<<148, 256, 0, st>>>(m_k, l_k, n, 1e30f, 1.0f);
        return ATT3_OK;
    }
    if ((rc = att3::dense_gather_forward(R, Q, S, Vq1, Vs1, mask, Yr, m_j, l_j, B, H, N, D, n_valid, st))) return rc;
    if ((rc = att3::dense_gather_forward(S, Q, R, Vq1, Vr1, mask, Ys, m_k, l_k, B, H, N, D, n_valid, st))) return rc;
    att3::count_launch(2, 2);
    if (scatter) {
        // each output weights a cell with the two softmaxes anchored at the other indices (cuda/forward.cu:941-1249)
        const ScatterSide q{Q, Vq2, m_i, l_i}, r{R, Vr2, m_j, l_j}, s{S, Vs2, m_k, l_k};
        if ((rc = scatter_forward(q, r, s, mask, Yq_, B, H, N, D, n_valid, st))) return rc;
        if ((rc = scatter_forward(r, q, s, mask, Yr_, B, H, N, D, n_valid, st))) return rc;
        if ((rc = scatter_forward(s, q, r, mask, Ys_, B, H, N, D, n_valid, st))) return rc;
        att3::count_launch(2, 3);
    }
    return ATT3_OK;
}

// ---------------------------------------------------------------------------------------------
// Three-gather backward
// ---------------------------------------------------------------------------------------------

// nine FP32 gradient planes + one anchor-gradient partial plane per 128-key tile
extern "C" size_t att3_hg_backward_workspace_bytes(int B, int H, int N, int D) {
    if (B <= 0 || H <= 0 || N <= 0 || D <= 0) return 0;
    const size_t plane = static_cast<size_t>(B) * H * N * D * sizeof(float);
    // the scatter terms use three planes of the same scratch area; two more for the anchor chunks of short sequences
    return plane * (9 + std::max(att3::dense_tiles(N, 0), 3) + 2);
}

extern "C" int att3_hg_backward(const void* gYq, const void* gYr, const void* gYs, const void* gYq_,
                                const void* gYr_, const void* gYs_, const void* Q, const void* R, const void* S,
                                const void* Vq1, const void* Vq2, const void* Vr1, const void* Vr2, const void* Vs1,
                                const void* Vs2, const void* Yq, const void* Yr, const void* Ys, const float* m_i,
                                const float* l_i, const float* m_j, const float* l_j, const float* m_k,
                                const float* l_k, const uint8_t* mask, void* dQ, void* dR, void* dS, void* dVq1,
                                void* dVq2, void* dVr1, void* dVr2, void* dVs1, void* dVs2, int B, int H, int N,
                                int D, int n_valid, int gather_mode, int scatter, void* workspace,
                                size_t workspace_bytes, void* stream) {
    if (int rc = check_hg("att3_hg_backward", B, H, N, D)) return rc;
    if (!gYq || !Q || !R || !S || !Vq1 || !Vr1 || !Vs1 || !Yq || !m_i || !l_i || !dQ || !dR || !dS || !dVq1 || !dVq2 ||
        !dVr1 || !dVr2 || !dVs1 || !dVs2)
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_backward: null tensor pointer");
    if (gather_mode == 0 && (!gYr || !gYs || !Yr || !Ys || !m_j || !l_j || !m_k || !l_k))
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_backward: null tensor pointer (R/S-anchored gathers)");
    if (!att3::require_sm100("att3_hg_backward")) return ATT3_ERR_UNSUPPORTED;
    if (scatter && (gather_mode != 0 || !gYq_ || !gYr_ || !gYs_ || !Vq2 || !Vr2 || !Vs2))
        return att3::set_error(ATT3_ERR_INVALID,
                               "att3_hg_backward: scatter gradients need gather_mode 0, the three scatter cotangents "
                               "and the second value tensors");
    const size_t need = att3_hg_backward_workspace_bytes(B, H, N, D);
    if (!workspace || workspace_bytes < need)
        return att3::set_error(ATT3_ERR_WORKSPACE, "att3_hg_backward: workspace of %zu bytes required, got %zu", need,
                               workspace_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t plane = static_cast<size_t>(B) * H * N * D;
    const int nt = att3::dense_tiles(N, n_valid);
    float* ws = static_cast<float*>(workspace);
    float *gQ = ws, *gR = ws + plane, *gS = ws + 2 * plane, *gVq1 = ws + 3 * plane, *gVq2 = ws + 4 * plane,
          *gVr1 = ws + 5 * plane, *gVr2 = ws + 6 * plane, *gVs1 = ws + 7 * plane, *gVs2 = ws + 8 * plane,
          *part = ws + 9 * plane, *chunk_scratch = part + static_cast<size_t>(std::max(att3::dense_tiles(N, 0), 3)) * plane;
    cudaMemsetAsync(ws, 0, 9 * plane * sizeof(float), st);

    // One anchored gather: anchor A with statistics (m,l), rows (Kr,Vr), cols (Kc,Vc).
    auto gather_bwd = [&](const void* A, const void* gY, const void* Y, const float* m, const float* l, const void* Kr,
                          const void* Vr, const void* Kc, const void* Vc, float* gA, float* gKr, float* gVr, float* gKc,
                          float* gVc) -> int {
        cudaMemsetAsync(part, 0, static_cast<size_t>(nt) * plane * sizeof(float), st);
        int rc = att3::dense_gather_backward_side(A, gY, Y, m, l, Kr, Vr, Kc, Vc, mask, gKc, gVc, part, B, H, N, D,
                                                  n_valid, st, chunk_scratch);
        if (rc) return rc;
        if ((rc = att3::add_planes(part, nt, plane, gA, st))) return rc;
        rc = att3::dense_gather_backward_side(A, gY, Y, m, l, Kc, Vc, Kr, Vr, mask, gKr, gVr, nullptr, B, H, N, D,
                                              n_valid, st, chunk_scratch);
        att3::count_launch(3, 3);
        return rc;
    };
    int rc = gather_bwd(Q, gYq, Yq, m_i, l_i, R, Vr1, S, Vs1, gQ, gR, gVr1, gS, gVs1);
    if (rc) return rc;
    if (gather_mode == 0) {
        if ((rc = gather_bwd(R, gYr, Yr, m_j, l_j, Q, Vq1, S, Vs1, gR, gQ, gVq1, gS, gVs1))) return rc;
        if ((rc = gather_bwd(S, gYs, Ys, m_k, l_k, Q, Vq1, R, Vr1, gS, gQ, gVq1, gR, gVr1))) return rc;
    }
    if (scatter) {
        const ScatterSide q{Q, Vq2, m_i, l_i}, r{R, Vr2, m_j, l_j}, s{S, Vs2, m_k, l_k};
        if ((rc = scatter_backward(q, r, s, gYq_, mask, gQ, gR, gS, gVr2, gVs2, part, B, H, N, D, n_valid, st))) return rc;
        if ((rc = scatter_backward(r, q, s, gYr_, mask, gR, gQ, gS, gVq2, gVs2, part, B, H, N, D, n_valid, st))) return rc;
        if ((rc = scatter_backward(s, q, r, gYs_, mask, gS, gQ, gR, gVq2, gVr2, part, B, H, N, D, n_valid, st))) return rc;
        att3::count_launch(3, 18);
    }
    void* outs[9] = {dQ, dR, dS, dVq1, dVq2, dVr1, dVr2, dVs1, dVs2};
    const float* srcs[9] = {gQ, gR, gS, gVq1, gVq2, gVr1, gVr2, gVs1, gVs2};
    for (int k = 0; k < 9; ++k)
        if ((rc = att3::plane_to_bf16(srcs[k], outs[k], plane, st))) return rc;
    return ATT3_OK;
}
