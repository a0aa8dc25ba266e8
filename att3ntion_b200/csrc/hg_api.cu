// Dense anchored-gather launchers and the C-ABI entry points of the three-gather
// hypergraph attention, which is three anchored gathers with permuted roles
// (forward) and the sum of their gradients (backward).
#include <algorithm>
#include <cmath>

#include "att3_abi_internal.h"
#include "ag_dense_bwd.cuh"

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

template <int DP, bool SC = false>
int launch_fwd(const agdense::FwdParams& p, cudaStream_t st) {
    using L = agdense::FwdSmem<DP>;
    if (int rc = opt_in_smem(agdense::ag_dense_fwd_kernel<DP, SC>, L::ALLOC, "dense gather forward: shared-memory opt-in")) return rc;
    dim3 grid((p.NA + p.group - 1) / p.group, p.H, p.B);
    att3::TimedLaunch timed(att3::K_DENSE_FWD, st);
    agdense::ag_dense_fwd_kernel<DP, SC><<<grid, agdense::NTHREADS, L::ALLOC, st>>>(p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ATT3_OK : att3::set_cuda_error(e, "dense gather forward: launch");
}

template <int DP, bool WITH_DA, int SC = 0>
int launch_bwd(const agdense::BwdParams& p, int n_tiles, cudaStream_t st) {
    using L = agdense::BwdSmem<DP, WITH_DA>;
    if (int rc = opt_in_smem(agdense::ag_dense_bwd_kernel<DP, WITH_DA, SC>, L::ALLOC, "dense gather backward: shared-memory opt-in"))
        return rc;
    dim3 grid(n_tiles * p.a_chunks, p.H, p.B);
    att3::TimedLaunch timed(att3::K_DENSE_BWD, st);
    agdense::ag_dense_bwd_kernel<DP, WITH_DA, SC><<<grid, agdense::BWD_THREADS, L::ALLOC, st>>>(p);
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

static agdense::FwdParams fwd_params(const void* A, const void* Rw, const void* C, const void* Vrow, const void* Vcol,
                                     const uint8_t* mask, void* Y, float* m, float* l, int B, int H, int D, Axis a,
                                     Axis r, Axis c) {
    agdense::FwdParams p{};
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.Rw = static_cast<const __nv_bfloat16*>(Rw);
    p.C = static_cast<const __nv_bfloat16*>(C);
    p.Vrow = static_cast<const __nv_bfloat16*>(Vrow);
    p.Vcol = static_cast<const __nv_bfloat16*>(Vcol);
    p.mask = mask;
    p.Y = static_cast<__nv_bfloat16*>(Y);
    p.m = m; p.l = l;
    p.B = B; p.H = H; p.D = D;
    p.NA = a.n; p.NR = r.n; p.NC = c.n;
    p.a_valid = a.valid; p.r_valid = r.valid; p.c_valid = c.valid;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = ag_status_ptr();
    // anchors per CTA: enough CTAs to fill the device twice over, at most 16 anchors each
    const long ctas_at_16 = static_cast<long>((a.n + 15) / 16) * H * B;
    p.group = ctas_at_16 >= 2L * sm_count() ? 16 : (ctas_at_16 * 2 >= 2L * sm_count() ? 8 : 4);
    return p;
}

int dense_gather_forward_axes(const void* A, const void* Rw, const void* C, const void* Vrow, const void* Vcol,
                              const uint8_t* mask, void* Y, float* m, float* l, int B, int H, int D, Axis a, Axis r,
                              Axis c, cudaStream_t st) {
    const agdense::FwdParams p = fwd_params(A, Rw, C, Vrow, Vcol, mask, Y, m, l, B, H, D, a, r, c);
    return D > 64 ? launch_fwd<128>(p, st) : launch_fwd<64>(p, st);
}

int dense_gather_forward(const void* A, const void* Rw, const void* C, const void* Vrow, const void* Vcol,
                         const uint8_t* mask, void* Y, float* m, float* l, int B, int H, int N, int D, int n_valid,
                         cudaStream_t st) {
    const Axis ax{N, n_valid};
    return dense_gather_forward_axes(A, Rw, C, Vrow, Vcol, mask, Y, m, l, B, H, D, ax, ax, ax, st);
}

// One scatter output: anchor = the output index, rows / cols = the two other indices with their second value
// tensors and the statistics of the softmaxes anchored at them.
int dense_scatter_forward(const void* A, const void* Rw, const void* C, const void* Vrow2, const void* Vcol2,
                          const float* m_row, const float* l_row, const float* m_col, const float* l_col,
                          const uint8_t* mask, void* out, int B, int H, int N, int D, int n_valid, cudaStream_t st) {
    const Axis ax{N, n_valid};
    agdense::FwdParams p = fwd_params(A, Rw, C, Vrow2, Vcol2, mask, out, nullptr, nullptr, B, H, D, ax, ax, ax);
    p.m_row = m_row; p.l_row = l_row; p.m_col = m_col; p.l_col = l_col;
    return D > 64 ? launch_fwd<128, true>(p, st) : launch_fwd<64, true>(p, st);
}

int dense_gather_backward_side(const void* A, const void* dY, const void* Y, const float* m, const float* l,
                               const void* Ka, const void* Va, const void* Kb, const void* Vb, const uint8_t* mask,
                               float* dKb, float* dVb, float* dA_part, int B, int H, int N, int D, int n_valid,
                               cudaStream_t st, float* chunk_scratch) {
    const Axis ax{N, n_valid};
    return dense_gather_backward_side_axes(A, dY, Y, m, l, Ka, Va, Kb, Vb, mask, dKb, dVb, dA_part, B, H, D, ax, ax, ax,
                                           st, chunk_scratch);
}

// own: the side whose gradients this launch produces (Kb, Vb); oth: the other key side (Ka, Va).
int dense_gather_backward_side_axes(const void* A, const void* dY, const void* Y, const float* m, const float* l,
                                    const void* Ka, const void* Va, const void* Kb, const void* Vb,
                                    const uint8_t* mask, float* dKb, float* dVb, float* dA_part, int B, int H, int D,
                                    Axis a, Axis own, Axis oth, cudaStream_t st, float* chunk_scratch) {
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
    p.B = B; p.H = H; p.D = D;
    p.NA = a.n; p.N_own = own.n; p.N_oth = oth.n;
    p.a_valid = a.valid; p.own_valid = own.valid; p.oth_valid = oth.valid;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = ag_status_ptr();
    const int nt = dense_tiles(own.n, own.valid);
    // One CTA per (own tile, batch, head) leaves most SMs idle for short sequences: split the anchors in two
    // when that still fits the machine and the caller has given room for the second chunk's planes.
    const size_t plane = static_cast<size_t>(B) * H * own.n * D;
    p.a_chunks = (chunk_scratch && 2 * nt * B * H <= sm_count() && a.n >= 2) ? 2 : 1;
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

// One pass of a scatter output's backward for one own side (pass 1: second-value gradient into `out_own`;
// pass 2: key gradient into `out_own` and, with dA_part, the anchor-gradient partial planes).
int dense_scatter_backward_side(int pass, const void* A, const void* G, const void* K_oth, const void* V2_oth,
                                const void* K_own, const void* V2_own, const float* m_own, const float* l_own,
                                const float* m_oth, const float* l_oth, const float* C_own, const float* C_oth,
                                const uint8_t* mask, float* out_own, float* dA_part, int B, int H, int N, int D,
                                int n_valid, cudaStream_t st, float* chunk_scratch) {
    agdense::BwdParams p{};
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.dY = static_cast<const __nv_bfloat16*>(G);
    p.Y = p.dY;                       // not read by the scatter passes
    p.Ka = static_cast<const __nv_bfloat16*>(K_oth);
    p.Va = static_cast<const __nv_bfloat16*>(V2_oth);
    p.Kb = static_cast<const __nv_bfloat16*>(K_own);
    p.Vb = static_cast<const __nv_bfloat16*>(V2_own);
    p.mask = mask;
    p.dKb = out_own; p.dVb = out_own; p.dA_part = dA_part;
    p.m_own = m_own; p.l_own = l_own; p.m_oth = m_oth; p.l_oth = l_oth; p.C_own = C_own; p.C_oth = C_oth;
    p.B = B; p.H = H; p.D = D;
    p.NA = p.N_own = p.N_oth = N;
    p.a_valid = p.own_valid = p.oth_valid = n_valid;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = ag_status_ptr();
    const int nt = dense_tiles(N, n_valid);
    const size_t plane = static_cast<size_t>(B) * H * N * D;
    p.a_chunks = (chunk_scratch && 2 * nt * B * H <= sm_count() && N >= 2) ? 2 : 1;
    p.dKb1 = chunk_scratch; p.dVb1 = chunk_scratch;
    if (p.a_chunks == 2) cudaMemsetAsync(chunk_scratch, 0, plane * sizeof(float), st);
    int rc;
    if (pass == 1) rc = D > 64 ? launch_bwd<128, false, 1>(p, nt, st) : launch_bwd<64, false, 1>(p, nt, st);
    else if (dA_part) rc = D > 64 ? launch_bwd<128, true, 2>(p, nt, st) : launch_bwd<64, true, 2>(p, nt, st);
    else rc = D > 64 ? launch_bwd<128, false, 2>(p, nt, st) : launch_bwd<64, false, 2>(p, nt, st);
    if (rc || p.a_chunks == 1) return rc;
    return add_planes(chunk_scratch, 1, plane, out_own, st);
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
// Scatter terms: the dense kernels in their scatter forms (tensor cores)
// ---------------------------------------------------------------------------------------------

// One index of the operator in a given role: its keys, second value tensor and the statistics of the
// softmax anchored at it.
struct ScatterSide {
    const void* keys; const void* v2; const float* m; const float* l;
};

// out[a] = sum_{u,v} Pu Pv Vu2[u] o Vv2[v]   (forward of one scatter output)
static int scatter_forward(const ScatterSide& a, const ScatterSide& u, const ScatterSide& v, const uint8_t* mask,
                           void* out, int B, int H, int N, int D, int n_valid, cudaStream_t st) {
    return att3::dense_scatter_forward(a.keys, u.keys, v.keys, u.v2, v.v2, u.m, u.l, v.m, v.l, mask, out, B, H, N, D,
                                       n_valid, st);
}

// Gradients of one scatter output under the cotangent g: into the FP32 planes of the three key tensors and
// of the two second value tensors.  tmp: two planes (this term's value gradients), one plane holding the two
// [B,H,N] correction vectors, and one anchor-gradient partial plane per 128-key tile.
static int scatter_backward(const ScatterSide& a, const ScatterSide& u, const ScatterSide& v, const void* g,
                            const uint8_t* mask, float* gA, float* gU, float* gV, float* gVu2, float* gVv2,
                            float* tmp, float* chunk_scratch, int B, int H, int N, int D, int n_valid,
                            cudaStream_t st) {
    const size_t plane = static_cast<size_t>(B) * H * N * D, rows = static_cast<size_t>(B) * H * N;
    const int nt = att3::dense_tiles(N, n_valid);
    float *tmpU = tmp, *tmpV = tmp + plane, *Cu = tmp + 2 * plane, *Cv = Cu + rows, *part = tmp + 3 * plane;
    cudaMemsetAsync(tmp, 0, 2 * plane * sizeof(float), st);
    int rc;
    // pass 1: value gradients of this term alone (their row dots are the softmax corrections of pass 2)
    if ((rc = att3::dense_scatter_backward_side(1, a.keys, g, v.keys, v.v2, u.keys, u.v2, u.m, u.l, v.m, v.l, nullptr,
                                                nullptr, mask, tmpU, nullptr, B, H, N, D, n_valid, st, chunk_scratch)))
        return rc;
    if ((rc = att3::dense_scatter_backward_side(1, a.keys, g, u.keys, u.v2, v.keys, v.v2, v.m, v.l, u.m, u.l, nullptr,
                                                nullptr, mask, tmpV, nullptr, B, H, N, D, n_valid, st, chunk_scratch)))
        return rc;
    const int wpb = 8;    // warps per block of the row-dot kernel
    const unsigned nblk = static_cast<unsigned>((rows + wpb - 1) / wpb);
    {
        att3::TimedLaunch timed(att3::K_HG_AUX, st);
        agdense::rowdot_kernel<<<nblk, wpb * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(u.v2), tmpU, Cu, rows, D);
    }
    {
        att3::TimedLaunch timed(att3::K_HG_AUX, st);
        agdense::rowdot_kernel<<<nblk, wpb * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(v.v2), tmpV, Cv, rows, D);
    }
    if ((rc = att3::add_planes(tmpU, 1, plane, gVu2, st))) return rc;
    if ((rc = att3::add_planes(tmpV, 1, plane, gVv2, st))) return rc;
    // pass 2: key gradients; the launch with own = u also produces the anchor gradient
    cudaMemsetAsync(part, 0, static_cast<size_t>(nt) * plane * sizeof(float), st);
    if ((rc = att3::dense_scatter_backward_side(2, a.keys, g, v.keys, v.v2, u.keys, u.v2, u.m, u.l, v.m, v.l, Cu, Cv,
                                                mask, gU, part, B, H, N, D, n_valid, st, chunk_scratch)))
        return rc;
    if ((rc = att3::add_planes(part, nt, plane, gA, st))) return rc;
    if ((rc = att3::dense_scatter_backward_side(2, a.keys, g, u.keys, u.v2, v.keys, v.v2, v.m, v.l, u.m, u.l, Cv, Cu,
                                                mask, gV, nullptr, B, H, N, D, n_valid, st, chunk_scratch)))
        return rc;
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

// Lengths I, J, K of the Q, R, S axes and how many leading entries of each are real.  The scatter outputs and a mask
// need equal lengths, as in the reference (cuda/forward.cu:1292, 1545).
static int check_axes(const char* who, int B, int H, int I, int J, int K, int D, bool has_mask, int scatter) {
    if (int rc = check_hg(who, B, H, I, D)) return rc;
    if (int rc = check_hg(who, B, H, J, D)) return rc;
    if (int rc = check_hg(who, B, H, K, D)) return rc;
    if (has_mask && !(I == J && J == K))
        return att3::set_error(ATT3_ERR_INVALID, "%s: a mask requires I == J == K, got %d, %d, %d", who, I, J, K);
    if (scatter && !(I == J && J == K))
        return att3::set_error(ATT3_ERR_INVALID, "%s: scatter requires I == J == K, got %d, %d, %d", who, I, J, K);
    return ATT3_OK;
}

static int axis_valid(int valid, int n) { return (valid > 0 && valid < n) ? valid : 0; }

extern "C" int att3_hg_forward_axes(const void* Q, const void* R, const void* S, const void* Vq1, const void* Vq2,
                                    const void* Vr1, const void* Vr2, const void* Vs1, const void* Vs2,
                                    const uint8_t* mask, void* Yq, void* Yr, void* Ys, void* Yq_, void* Yr_, void* Ys_,
                                    float* m_i, float* l_i, float* m_j, float* l_j, float* m_k, float* l_k, int B,
                                    int H, int I, int J, int K, int D, int I_valid, int J_valid, int K_valid,
                                    int gather_mode, int scatter, void* stream) {
    if (int rc = check_axes("att3_hg_forward", B, H, I, J, K, D, mask != nullptr, scatter)) return rc;
    if (!Q || !R || !S || !Vq1 || !Vr1 || !Vs1 || !Yq || !Yr || !Ys || !Yq_ || !Yr_ || !Ys_ || !m_i || !l_i || !m_j ||
        !l_j || !m_k || !l_k)
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_forward: null tensor pointer");
    if (gather_mode != 0 && gather_mode != 1)
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_forward: gather_mode must be 0 or 1, got %d", gather_mode);
    if (scatter && gather_mode != 0)
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_forward: scatter needs all three gathers (gather_mode 0)");
    if (scatter && (!Vq2 || !Vr2 || !Vs2))
        return att3::set_error(ATT3_ERR_INVALID, "att3_hg_forward: scatter needs the second value tensors");
    const int vi = axis_valid(I_valid, I), vj = axis_valid(J_valid, J), vk = axis_valid(K_valid, K);
    if (scatter && !(vi == vj && vj == vk))
        return att3::set_error(ATT3_ERR_UNSUPPORTED, "att3_hg_forward: scatter takes one valid length for the three axes");
    if (!att3::require_sm100("att3_hg_forward")) return ATT3_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const att3::Axis ai{I, vi}, aj{J, vj}, ak{K, vk};
    const size_t ni = static_cast<size_t>(B) * H * I, nj = static_cast<size_t>(B) * H * J, nk = static_cast<size_t>(B) * H * K;
    // outputs of skipped gathers / scatters read as zero (cuda/forward.cu:1308-1321)
    cudaMemsetAsync(Yq_, 0, ni * D * 2, st);
    cudaMemsetAsync(Yr_, 0, nj * D * 2, st);
    cudaMemsetAsync(Ys_, 0, nk * D * 2, st);
    int rc = att3::dense_gather_forward_axes(Q, R, S, Vr1, Vs1, mask, Yq, m_i, l_i, B, H, D, ai, aj, ak, st);
    if (rc) return rc;
    att3::count_launch(2);
    if (gather_mode == 1) {
        cudaMemsetAsync(Yr, 0, nj * D * 2, st);
        cudaMemsetAsync(Ys, 0, nk * D * 2, st);
        // statistics that make the other two softmax weights vanish (cuda/forward.cu:1455-1459)
        fill_stats_kernel<<<148, 256, 0, st>>>(m_j, l_j, nj, 1e30f, 1.0f);
        fill_stats_kernel<<<148, 256, 0, st>>>(m_k, l_k, nk, 1e30f, 1.0f);
        return ATT3_OK;
    }
    if ((rc = att3::dense_gather_forward_axes(R, Q, S, Vq1, Vs1, mask, Yr, m_j, l_j, B, H, D, aj, ai, ak, st))) return rc;
    if ((rc = att3::dense_gather_forward_axes(S, Q, R, Vq1, Vr1, mask, Ys, m_k, l_k, B, H, D, ak, ai, aj, st))) return rc;
    att3::count_launch(2, 2);
    if (scatter) {
        // each output weights a cell with the two softmaxes anchored at the other indices (cuda/forward.cu:941-1249)
        const int N = I, n_valid = vi;
        const ScatterSide q{Q, Vq2, m_i, l_i}, r{R, Vr2, m_j, l_j}, s{S, Vs2, m_k, l_k};
        if ((rc = scatter_forward(q, r, s, mask, Yq_, B, H, N, D, n_valid, st))) return rc;
        if ((rc = scatter_forward(r, q, s, mask, Yr_, B, H, N, D, n_valid, st))) return rc;
        if ((rc = scatter_forward(s, q, r, mask, Ys_, B, H, N, D, n_valid, st))) return rc;
        att3::count_launch(2, 3);
    }
    return ATT3_OK;
}

extern "C" int att3_hg_forward(const void* Q, const void* R, const void* S, const void* Vq1, const void* Vq2,
                               const void* Vr1, const void* Vr2, const void* Vs1, const void* Vs2,
                               const uint8_t* mask, void* Yq, void* Yr, void* Ys, void* Yq_, void* Yr_, void* Ys_,
                               float* m_i, float* l_i, float* m_j, float* l_j, float* m_k, float* l_k, int B, int H,
                               int N, int D, int n_valid, int gather_mode, int scatter, void* stream) {
    return att3_hg_forward_axes(Q, R, S, Vq1, Vq2, Vr1, Vr2, Vs1, Vs2, mask, Yq, Yr, Ys, Yq_, Yr_, Ys_, m_i, l_i, m_j, l_j,
                                m_k, l_k, B, H, N, N, N, D, n_valid, n_valid, n_valid, gather_mode, scatter, stream);
}

// ---------------------------------------------------------------------------------------------
// Three-gather backward
// ---------------------------------------------------------------------------------------------

// Nine FP32 gradient planes + one anchor-gradient partial plane per 128-key tile, each plane sized for the longest of
// the three axes.
extern "C" size_t att3_hg_backward_axes_workspace_bytes(int B, int H, int I, int J, int K, int D) {
    if (B <= 0 || H <= 0 || I <= 0 || J <= 0 || K <= 0 || D <= 0) return 0;
    const int N = std::max(I, std::max(J, K));
    const size_t plane = static_cast<size_t>(B) * H * N * D * sizeof(float);
    // the scatter terms use three more planes next to the partial planes; two more for the anchor chunks of short sequences
    return plane * (9 + att3::dense_tiles(N, 0) + 3 + 2);
}

extern "C" size_t att3_hg_backward_workspace_bytes(int B, int H, int N, int D) {
    return att3_hg_backward_axes_workspace_bytes(B, H, N, N, N, D);
}

extern "C" int att3_hg_backward_axes(const void* gYq, const void* gYr, const void* gYs, const void* gYq_,
                                     const void* gYr_, const void* gYs_, const void* Q, const void* R, const void* S,
                                     const void* Vq1, const void* Vq2, const void* Vr1, const void* Vr2,
                                     const void* Vs1, const void* Vs2, const void* Yq, const void* Yr, const void* Ys,
                                     const float* m_i, const float* l_i, const float* m_j, const float* l_j,
                                     const float* m_k, const float* l_k, const uint8_t* mask, void* dQ, void* dR,
                                     void* dS, void* dVq1, void* dVq2, void* dVr1, void* dVr2, void* dVs1, void* dVs2,
                                     int B, int H, int I, int J, int K, int D, int I_valid, int J_valid, int K_valid,
                                     int gather_mode, int scatter, void* workspace, size_t workspace_bytes,
                                     void* stream) {
    if (int rc = check_axes("att3_hg_backward", B, H, I, J, K, D, mask != nullptr, scatter)) return rc;
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
    const int vi = axis_valid(I_valid, I), vj = axis_valid(J_valid, J), vk = axis_valid(K_valid, K);
    if (scatter && !(vi == vj && vj == vk))
        return att3::set_error(ATT3_ERR_UNSUPPORTED, "att3_hg_backward: scatter takes one valid length for the three axes");
    const size_t need = att3_hg_backward_axes_workspace_bytes(B, H, I, J, K, D);
    if (!workspace || workspace_bytes < need)
        return att3::set_error(ATT3_ERR_WORKSPACE, "att3_hg_backward: workspace of %zu bytes required, got %zu", need,
                               workspace_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const att3::Axis ai{I, vi}, aj{J, vj}, ak{K, vk};
    const int Nmax = std::max(I, std::max(J, K));
    const size_t plane = static_cast<size_t>(B) * H * Nmax * D;      // capacity of a workspace plane
    const size_t len_i = static_cast<size_t>(B) * H * I * D, len_j = static_cast<size_t>(B) * H * J * D,
                 len_k = static_cast<size_t>(B) * H * K * D;         // what each tensor's gradient uses of it
    float* ws = static_cast<float*>(workspace);
    float *gQ = ws, *gR = ws + plane, *gS = ws + 2 * plane, *gVq1 = ws + 3 * plane, *gVq2 = ws + 4 * plane,
          *gVr1 = ws + 5 * plane, *gVr2 = ws + 6 * plane, *gVs1 = ws + 7 * plane, *gVs2 = ws + 8 * plane,
          *part = ws + 9 * plane, *chunk_scratch = part + static_cast<size_t>(att3::dense_tiles(Nmax, 0) + 3) * plane;
    cudaMemsetAsync(ws, 0, 9 * plane * sizeof(float), st);

    // One anchored gather: anchor A (axis a, gradient length len_a) with statistics (m,l), rows (Kr,Vr; axis r),
    // cols (Kc,Vc; axis c).
    auto gather_bwd = [&](const void* A, const void* gY, const void* Y, const float* m, const float* l, const void* Kr,
                          const void* Vr, const void* Kc, const void* Vc, float* gA, float* gKr, float* gVr, float* gKc,
                          float* gVc, att3::Axis a, att3::Axis r, att3::Axis c, size_t len_a) -> int {
        const int nt = att3::dense_tiles(c.n, c.valid);
        cudaMemsetAsync(part, 0, static_cast<size_t>(nt) * len_a * sizeof(float), st);
        int rc = att3::dense_gather_backward_side_axes(A, gY, Y, m, l, Kr, Vr, Kc, Vc, mask, gKc, gVc, part, B, H, D, a,
                                                       c, r, st, chunk_scratch);
        if (rc) return rc;
        if ((rc = att3::add_planes(part, nt, len_a, gA, st))) return rc;
        rc = att3::dense_gather_backward_side_axes(A, gY, Y, m, l, Kc, Vc, Kr, Vr, mask, gKr, gVr, nullptr, B, H, D, a,
                                                   r, c, st, chunk_scratch);
        att3::count_launch(3, 3);
        return rc;
    };
    int rc = gather_bwd(Q, gYq, Yq, m_i, l_i, R, Vr1, S, Vs1, gQ, gR, gVr1, gS, gVs1, ai, aj, ak, len_i);
    if (rc) return rc;
    if (gather_mode == 0) {
        if ((rc = gather_bwd(R, gYr, Yr, m_j, l_j, Q, Vq1, S, Vs1, gR, gQ, gVq1, gS, gVs1, aj, ai, ak, len_j))) return rc;
        if ((rc = gather_bwd(S, gYs, Ys, m_k, l_k, Q, Vq1, R, Vr1, gS, gQ, gVq1, gR, gVr1, ak, ai, aj, len_k))) return rc;
    }
    if (scatter) {
        const int N = I, n_valid = vi;
        const ScatterSide q{Q, Vq2, m_i, l_i}, r{R, Vr2, m_j, l_j}, s{S, Vs2, m_k, l_k};
        if ((rc = scatter_backward(q, r, s, gYq_, mask, gQ, gR, gS, gVr2, gVs2, part, chunk_scratch, B, H, N, D, n_valid, st))) return rc;
        if ((rc = scatter_backward(r, q, s, gYr_, mask, gR, gQ, gS, gVq2, gVs2, part, chunk_scratch, B, H, N, D, n_valid, st))) return rc;
        if ((rc = scatter_backward(s, q, r, gYs_, mask, gS, gQ, gR, gVq2, gVr2, part, chunk_scratch, B, H, N, D, n_valid, st))) return rc;
        att3::count_launch(3, 12);
    }
    void* outs[9] = {dQ, dR, dS, dVq1, dVq2, dVr1, dVr2, dVs1, dVs2};
    const float* srcs[9] = {gQ, gR, gS, gVq1, gVq2, gVr1, gVr2, gVs1, gVs2};
    const size_t lens[9] = {len_i, len_j, len_k, len_i, len_i, len_j, len_j, len_k, len_k};
    for (int k = 0; k < 9; ++k)
        if ((rc = att3::plane_to_bf16(srcs[k], outs[k], lens[k], st))) return rc;
    return ATT3_OK;
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
    return att3_hg_backward_axes(gYq, gYr, gYs, gYq_, gYr_, gYs_, Q, R, S, Vq1, Vq2, Vr1, Vr2, Vs1, Vs2, Yq, Yr, Ys, m_i,
                                 l_i, m_j, l_j, m_k, l_k, mask, dQ, dR, dS, dVq1, dVq2, dVr1, dVr2, dVs1, dVs2, B, H, N, N,
                                 N, D, n_valid, n_valid, n_valid, gather_mode, scatter, workspace, workspace_bytes, stream);
}
