// C-ABI entry points of the single query gather (independent and shared KV
// heads): argument validation, query-block partitioning and kernel launches.
#include <algorithm>
#include <atomic>
#include <cmath>

#include "att3_abi_internal.h"
#include "sg_ring_fwd.cuh"
#include "sg_ring_bwd.cuh"
#include "sg_pack_q.cuh"
#include "sg_pack_kv.cuh"

namespace {

// Sticky status word of this translation unit's kernels (bounded-wait failures).
__device__ int g_sg_status = 0;

// Device address of the status word on the current device.  The symbol is resolved once per
// device and thread (a thread-local table, so concurrent callers never share a slot that is
// being written); a failed look-up returns null and the entry point reports it.
int* status_ptr() {
    constexpr int kMaxDevices = 64;
    static thread_local int* cached[kMaxDevices] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!cached[dev]) {
        int* p = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_sg_status) != cudaSuccess) return nullptr;
        cached[dev] = p;
    }
    return cached[dev];
}

// Validation shared by forward and backward; mirrors single_gather_check and
// single_gather_shared_check of the reference (cuda/forward.cu:1609-1653).
int check_shapes(const char* who, int B, int Hq, int Hkv, int N, int D, int window, int q_begin) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0)
        return att3::set_error(ATT3_ERR_INVALID, "%s: empty batch/head dimensions are unsupported", who);
    if (N <= 0 || N % 16 != 0)
        return att3::set_error(ATT3_ERR_INVALID, "%s: N must be a positive multiple of 16, got %d", who, N);
    if (D != 64 && D != 128) return att3::set_error(ATT3_ERR_INVALID, "%s: D must be 64 or 128, got %d", who, D);
    if (Hq % Hkv != 0)
        return att3::set_error(ATT3_ERR_INVALID, "%s: Hq=%d is not divisible by Hkv=%d", who, Hq, Hkv);
    if (window < 0 || window > sgring::RING)
        return att3::set_error(ATT3_ERR_INVALID, "%s: window must be in [0,128], got %d", who, window);
    if (q_begin < 0 || q_begin >= N)
        return att3::set_error(ATT3_ERR_INVALID, "%s: q_begin must be in [0,N), got %d", who, q_begin);
    return ATT3_OK;
}

// Query-block partition of the ring kernels: as many CTAs as the device holds
// at `ctas_per_sm` residency, never shorter than `min_len` queries per block.
int plan_blocks(int B, int Hkv, int N, int q_begin, int sm_count, int ctas_per_sm, int min_len, int* block_len) {
    const int nq = N - q_begin;
    const int slots = std::max(1, sm_count * ctas_per_sm);
    int nblk = std::max(1, slots / std::max(1, B * Hkv));
    int len = (nq + nblk - 1) / nblk;
    len = std::max(len, std::min(min_len, nq));
    nblk = (nq + len - 1) / len;
    *block_len = len;
    return nblk;
}

// Schedule overrides (att3_sg_set_query_block): queries per CTA of the forward and of the backward
// passes, 0 = the built-in choice.
std::atomic<int> g_fwd_block{0}, g_bwd_block{0};

// Extensions of the current call (att3_sg_forward_ext / att3_sg_backward_ext set them around the regular entry
// point on the calling thread): the window of the S / Vs key axis when it differs from the R / Vr axis's, and the
// caller's mask as packed words.
struct SgExt { int window_s; const uint32_t* mask_words; int layout; void* Y_act; int precise; };
thread_local SgExt t_ext = {0, nullptr, 0, nullptr, 0};
int ext_window_s(int window) { return t_ext.window_s > 0 ? t_ext.window_s : window; }

// Packed schedule (sg_pack_q.cuh, sg_pack_kv.cuh): windows of at most 64 keys, D = 128, at least four query
// heads per KV head, q_begin a multiple of 8 (of every QB).  g_pack_off switches it off (schedule override).
std::atomic<int> g_pack_off{0};
bool pack_eligible(int Hq, int Hkv, int D, int window, int q_begin) {
    return !g_pack_off.load() && D == 128 && window >= 1 && window <= 64 && Hq / Hkv >= 4 && q_begin % 8 == 0 &&
           ext_window_s(window) == window && !t_ext.precise;     // equal windows on both key axes, plain products
}
int pack_slots(int window) { return window <= 16 ? 16 : window <= 32 ? 32 : 64; }
int round_up8(int v) { return (v + 7) / 8 * 8; }

// Backward partition: one block per SM where the problem allows it, blocks never shorter than
// BWD_MIN_BLOCK queries.  The block length is a function of (B, Hkv, N) only -- not of q_begin -- so
// that the workspace size, which depends on it through the number of partial planes, can be asked
// for without knowing where the caller's queries start.  (Many short blocks handed out by the
// hardware's CTA scheduler were measured instead: 32 queries per block, 1024 CTAs on 148 SMs, ran
// 2 % slower than the even split, 128 and 64 per block 12 % slower.)
int bwd_block_len(int B, int Hkv, int N) {
    if (const int v = g_bwd_block.load()) return std::max(v, sgring::BWD_MIN_BLOCK);
    int len = 0;
    plan_blocks(B, Hkv, N, 0, att3::sm_count(), 1, sgring::BWD_MIN_BLOCK, &len);
    return len;
}

}  // namespace

extern "C" int att3_sg_set_query_block(int fwd_len, int bwd_len) {
    if (fwd_len < 0 || bwd_len < 0 || (fwd_len && fwd_len < 16) || (bwd_len && bwd_len < sgring::BWD_MIN_BLOCK))
        return att3::set_error(ATT3_ERR_INVALID, "att3_sg_set_query_block: lengths must be 0 (automatic) or >= 16");
    g_fwd_block.store(fwd_len);
    g_bwd_block.store(bwd_len);
    return ATT3_OK;
}

extern "C" int att3_sg_set_packed(int on) {
    const int prev = g_pack_off.exchange(on ? 0 : 1);
    return prev ? 0 : 1;
}

extern "C" int att3_sg_query_blocks(int B, int Hq, int Hkv, int N, int q_begin, int sm_count, int* block_len) {
    (void)Hq;
    int len = 0;
    const int n = plan_blocks(B, Hkv, N, q_begin, sm_count, 1, 16, &len);     // the forward: one CTA per SM
    if (block_len) *block_len = len;
    return n * B * Hkv;
}

extern "C" int att3_device_status(void* stream) {
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_device_status: synchronize");
    int h = 0, h2 = 0;
    e = cudaMemcpyFromSymbol(&h, g_sg_status, sizeof(int));
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_device_status: read");
    if (int rc = att3::dense_status_read_and_clear(&h2)) return rc;
    if (h == 0) h = h2;
    if (h != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_sg_status, &zero, sizeof(int));
        return att3::set_error(ATT3_ERR_TIMEOUT, "a bounded device-side wait ran out (status %d)", h);
    }
    return ATT3_OK;
}

// A kernel whose only job is to let a bounded wait run out: one thread waits on an mbarrier that
// nobody ever arrives on, gives up after `limit` polls, records the fact in the status word and
// the kernel returns normally.  It is how the failure path (status word -> att3_device_status ->
// ATT3_ERR_TIMEOUT) is exercised without a fault, a trap or a hang.
__global__ void wait_selftest_kernel(int* status, unsigned limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        sm100::mbar_init(&bar, 1);
        sm100::fence_mbar_init();
        if (!sm100::mbar_wait(&bar, 0, limit)) atomicExch(status, 7);
        sm100::mbar_inval(&bar);
    }
}

extern "C" int att3_wait_selftest(unsigned limit, void* stream) {
    if (limit == 0 || limit > (1u << 20))
        return att3::set_error(ATT3_ERR_INVALID, "att3_wait_selftest: limit must be in [1, 2^20] polls");
    if (!att3::require_sm100("att3_wait_selftest")) return ATT3_ERR_UNSUPPORTED;
    int* st = status_ptr();
    if (!st) return att3::set_error(ATT3_ERR_CUDA, "att3_wait_selftest: status word not resolvable");
    wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(st, limit);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ATT3_OK : att3::set_cuda_error(e, "att3_wait_selftest: launch");
}

template <int D, bool EXT>
static int launch_ring_fwd(const sgring::FwdParams& p, int nblk, cudaStream_t stream) {
    using L = sgring::FwdSmem<D>;
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(sgring::sg_ring_fwd_kernel<D, EXT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, L::ALLOC);
        if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_forward: shared-memory opt-in");
        configured_dev = dev;
    }
    dim3 grid(nblk, p.Hkv, p.B);
    att3::TimedLaunch timed(att3::K_SG_FWD, stream);
    sgring::sg_ring_fwd_kernel<D, EXT><<<grid, sgring::PIPE_THREADS, L::ALLOC, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_forward: launch");
    att3::count_launch(0);
    return ATT3_OK;
}

template <int W, int MODE>
static int launch_pack_q(const sgpack::QParams& p, int nblk, cudaStream_t stream, const char* who) {
    using L = sgpack::QSmem<128, W, MODE>;
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(sgpack::sg_pack_q_kernel<128, W, MODE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, L::ALLOC);
        if (e != cudaSuccess) return att3::set_cuda_error(e, who);
        configured_dev = dev;
    }
    dim3 grid(nblk, p.Hkv, p.B);
    att3::TimedLaunch timed(MODE == sgpack::PQ_FWD ? att3::K_SG_FWD : att3::K_SG_BWD, stream);
    sgpack::sg_pack_q_kernel<128, W, MODE><<<grid, sgring::PIPE_THREADS, L::ALLOC, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return att3::set_cuda_error(e, who);
    att3::count_launch(MODE == sgpack::PQ_FWD ? 0 : 1);
    return ATT3_OK;
}

// Query-anchored packed kernel (forward, or dQ when dY is given) for a window of at most 64 keys.
static int run_pack_q(int mode, const void* Q, const void* R, const void* S, const void* Vr, const void* Vs,
                      const uint8_t* mask, void* Y, float* m, float* l, const void* dY, const float* delta, void* dQ,
                      int B, int Hq, int Hkv, int N, int window, int q_begin, int* status, cudaStream_t st,
                      const char* who) {
    const int W = pack_slots(window), QB = 128 / W, D = 128;
    sgpack::QParams p{};
    p.Q = static_cast<const __nv_bfloat16*>(Q);
    p.R = static_cast<const __nv_bfloat16*>(R);
    p.S = static_cast<const __nv_bfloat16*>(S);
    p.Vr = static_cast<const __nv_bfloat16*>(Vr);
    p.Vs = static_cast<const __nv_bfloat16*>(Vs);
    p.mask = mask;
    p.mask_words = t_ext.mask_words;
    if (mode == sgpack::PQ_FWD) {
        p.Y = static_cast<__nv_bfloat16*>(Y); p.m = m; p.l = l;
    } else {
        p.m_in = m; p.l_in = l; p.delta = delta; p.dQ = static_cast<__nv_bfloat16*>(dQ);
    }
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.N = N; p.window = window; p.q_begin = q_begin;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = status;
    p.bnhd = t_ext.layout;
    p.Y_act = mode == sgpack::PQ_FWD ? static_cast<__nv_bfloat16*>(t_ext.Y_act) : nullptr;
    int rc;
    if ((rc = att3::make_head_tensor_map(&p.tmQ, Q, B, Hq, N, D, p.bnhd, QB, who))) return rc;
    if (mode == sgpack::PQ_DQ && (rc = att3::make_head_tensor_map(&p.tmdY, dY, B, Hq, N, D, p.bnhd, QB, who))) return rc;
    if ((rc = att3::make_head_tensor_map(&p.tmR, R, B, Hkv, N, D, p.bnhd, QB, who))) return rc;
    if ((rc = att3::make_head_tensor_map(&p.tmVr, Vr, B, Hkv, N, D, p.bnhd, QB, who))) return rc;
    if ((rc = att3::make_head_tensor_map(&p.tmS, S, B, Hkv, N, D, p.bnhd, QB, who))) return rc;
    if ((rc = att3::make_head_tensor_map(&p.tmVs, Vs, B, Hkv, N, D, p.bnhd, QB, who))) return rc;
    int nblk = plan_blocks(B, Hkv, N, q_begin, att3::sm_count(), 1, 16, &p.block_len);
    if (const int forced = g_fwd_block.load()) p.block_len = forced;
    p.block_len = round_up8(p.block_len);
    nblk = (N - q_begin + p.block_len - 1) / p.block_len;
    const bool fwd = mode == sgpack::PQ_FWD;
    switch (W) {
        case 16: return fwd ? launch_pack_q<16, sgpack::PQ_FWD>(p, nblk, st, who) : launch_pack_q<16, sgpack::PQ_DQ>(p, nblk, st, who);
        case 32: return fwd ? launch_pack_q<32, sgpack::PQ_FWD>(p, nblk, st, who) : launch_pack_q<32, sgpack::PQ_DQ>(p, nblk, st, who);
        default: return fwd ? launch_pack_q<64, sgpack::PQ_FWD>(p, nblk, st, who) : launch_pack_q<64, sgpack::PQ_DQ>(p, nblk, st, who);
    }
}

extern "C" int att3_sg_forward(const void* Q, const void* R, const void* S, const void* Vr, const void* Vs,
                               const uint8_t* mask, void* Y, float* m, float* l, int B, int Hq, int Hkv, int N,
                               int D, int window, int q_begin, void* stream) {
    if (int rc = check_shapes("att3_sg_forward", B, Hq, Hkv, N, D, window, q_begin)) return rc;
    if (!Q || !R || !S || !Vr || !Vs || !Y || !m || !l)
        return att3::set_error(ATT3_ERR_INVALID, "att3_sg_forward: null tensor pointer");
    if (!att3::require_sm100("att3_sg_forward")) return ATT3_ERR_UNSUPPORTED;
    if (window == 0) {
        // every key a candidate: the dense anchored gather with (anchor, rows, cols) = (Q, R, S)
        if (Hkv != Hq)
            return att3::set_error(ATT3_ERR_UNSUPPORTED, "att3_sg_forward: shared KV heads need a window (1..128)");
        if (q_begin != 0) return att3::set_error(ATT3_ERR_INVALID, "att3_sg_forward: q_begin needs a window");
        att3::count_launch(0);
        return att3::dense_gather_forward(Q, R, S, Vr, Vs, mask, Y, m, l, B, Hq, N, D, 0,
                                          static_cast<cudaStream_t>(stream));
    }
    if (pack_eligible(Hq, Hkv, D, window, q_begin)) {
        int* status = status_ptr();
        if (!status) return att3::set_error(ATT3_ERR_CUDA, "att3_sg_forward: status word not resolvable");
        return run_pack_q(sgpack::PQ_FWD, Q, R, S, Vr, Vs, mask, Y, m, l, nullptr, nullptr, nullptr, B, Hq, Hkv, N, window,
                          q_begin, status, static_cast<cudaStream_t>(stream), "att3_sg_forward");
    }
    sgring::FwdParams p;
    p.Q = static_cast<const __nv_bfloat16*>(Q);
    p.R = static_cast<const __nv_bfloat16*>(R);
    p.S = static_cast<const __nv_bfloat16*>(S);
    p.Vr = static_cast<const __nv_bfloat16*>(Vr);
    p.Vs = static_cast<const __nv_bfloat16*>(Vs);
    p.mask = mask;
    p.mask_words = t_ext.mask_words;
    p.Y = static_cast<__nv_bfloat16*>(Y);
    p.m = m;
    p.l = l;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.N = N; p.window = window; p.q_begin = q_begin;
    p.window_s = ext_window_s(window);
    p.precise = t_ext.precise;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = status_ptr();
    if (!p.status) return att3::set_error(ATT3_ERR_CUDA, "att3_sg_forward: status word not resolvable");
    p.bnhd = t_ext.layout;
    p.Y_act = static_cast<__nv_bfloat16*>(t_ext.Y_act);
    {   // TMA descriptors for the kernel's row staging (one row per copy)
        int rc;
        if ((rc = att3::make_head_tensor_map(&p.tmQ, Q, B, Hq, N, D, p.bnhd, 1, "att3_sg_forward"))) return rc;
        if ((rc = att3::make_head_tensor_map(&p.tmR, R, B, Hkv, N, D, p.bnhd, 1, "att3_sg_forward"))) return rc;
        if ((rc = att3::make_head_tensor_map(&p.tmVr, Vr, B, Hkv, N, D, p.bnhd, 1, "att3_sg_forward"))) return rc;
        if ((rc = att3::make_head_tensor_map(&p.tmS, S, B, Hkv, N, D, p.bnhd, 1, "att3_sg_forward"))) return rc;
        if ((rc = att3::make_head_tensor_map(&p.tmVs, Vs, B, Hkv, N, D, p.bnhd, 1, "att3_sg_forward"))) return rc;
    }
    int nblk = plan_blocks(B, Hkv, N, q_begin, att3::sm_count(), 1, 16, &p.block_len);
    if (const int forced = g_fwd_block.load()) {
        p.block_len = forced;
        nblk = (N - q_begin + forced - 1) / forced;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the lean instantiation unless an extension is in use
    const bool ext = p.bnhd || p.Y_act || p.mask_words || p.window_s != p.window || p.precise;
    if (ext) return D == 64 ? launch_ring_fwd<64, true>(p, nblk, st) : launch_ring_fwd<128, true>(p, nblk, st);
    return D == 64 ? launch_ring_fwd<64, false>(p, nblk, st) : launch_ring_fwd<128, false>(p, nblk, st);
}

// ---------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------

// Workspace: FP32 partial planes of the two gradients of one key side (bwd_planes
// of them each); the second pass reuses the space after the first pass's reduction.
extern "C" size_t att3_sg_backward_workspace_bytes(int B, int Hq, int Hkv, int N, int D, int window) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || N <= 0 || D <= 0 || window < 0) return 0;
    if (window == 0)   // dense: five FP32 gradient planes + one anchor-gradient partial plane per 128-key tile
        return static_cast<size_t>(5 + att3::dense_tiles(N, 0) + 2) * B * Hq * N * D * sizeof(float);
    // partial planes of one key side, then delta = rowsum(dY o Y) per (batch, query head, query) for the packed schedule
    return static_cast<size_t>(2 * sgring::bwd_planes(bwd_block_len(B, Hkv, N))) * B * Hkv * N * D * sizeof(float) +
           static_cast<size_t>(B) * Hq * N * sizeof(float);
}

template <int D, bool WITH_DQ, bool EXT>
static int launch_ring_bwd_x(const sgring::BwdParams& p, int nblk, cudaStream_t stream) {
    using L = sgring::PipeSmem<D, WITH_DQ>;
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(sgring::sg_ring_bwd_kernel<D, WITH_DQ, EXT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, L::ALLOC);
        if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_backward: shared-memory opt-in");
        configured_dev = dev;
    }
    dim3 grid(nblk, p.Hkv, p.B);
    att3::TimedLaunch timed(att3::K_SG_BWD, stream);
    sgring::sg_ring_bwd_kernel<D, WITH_DQ, EXT><<<grid, sgring::PIPE_THREADS, L::ALLOC, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_backward: launch");
    att3::count_launch(1);
    return ATT3_OK;
}

template <int D, bool WITH_DQ>
static int launch_ring_bwd(const sgring::BwdParams& p, int nblk, cudaStream_t stream) {
    // the lean instantiation unless an extension is in use
    const bool ext = p.bnhd || p.mask_words || p.window_oth != p.window || p.precise;
    return ext ? launch_ring_bwd_x<D, WITH_DQ, true>(p, nblk, stream) : launch_ring_bwd_x<D, WITH_DQ, false>(p, nblk, stream);
}

static int launch_reduce(const sgring::BwdParams& p, int nblk, int D, void* dK, void* dV, cudaStream_t stream,
                         bool f32 = false, int lead = 0) {
    sgring::ReduceParams r;
    r.lead = lead;
    r.bnhd = t_ext.layout;
    r.Hkv = p.Hkv;
    r.part_K = p.part_K;
    r.part_V = p.part_V;
    r.dK = f32 ? nullptr : static_cast<__nv_bfloat16*>(dK);
    r.dV = f32 ? nullptr : static_cast<__nv_bfloat16*>(dV);
    r.dK32 = f32 ? static_cast<float*>(dK) : nullptr;
    r.dV32 = f32 ? static_cast<float*>(dV) : nullptr;
    r.rows = p.B * p.Hkv;
    r.N = p.N; r.D = D; r.q_begin = p.q_begin; r.block_len = p.block_len; r.nblk = nblk; r.planes = p.planes;
    const size_t total = static_cast<size_t>(r.rows) * p.N * (D / 4);
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<size_t>((total + threads - 1) / threads, 148 * 16));
    att3::TimedLaunch timed(att3::K_SG_REDUCE, stream);
    sgring::sg_bwd_reduce_kernel<<<blocks, threads, 0, stream>>>(r);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_backward: reduce launch");
    att3::count_launch(1);
    return ATT3_OK;
}

template <int W>
static int launch_pack_kv(const sgpack::KvParams& p, int nblk, cudaStream_t stream) {
    using L = sgpack::KvSmem<128, W>;
    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(sgpack::sg_pack_kv_kernel<128, W>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             L::ALLOC);
        if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_backward: shared-memory opt-in");
        configured_dev = dev;
    }
    dim3 grid(nblk, p.Hkv, p.B);
    att3::TimedLaunch timed(att3::K_SG_BWD, stream);
    sgpack::sg_pack_kv_kernel<128, W><<<grid, sgring::PIPE_THREADS, L::ALLOC, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_backward: launch");
    att3::count_launch(1);
    return ATT3_OK;
}

// delta[b,h,i] = sum_d dY o Y, the pre-pass of every windowed backward.
template <int D>
static int launch_delta(const void* dY, const void* Y, float* delta, int B, int Hq, int N, cudaStream_t st) {
    const size_t rows = static_cast<size_t>(B) * Hq * N;
    const int threads = 256;
    const unsigned blocks = static_cast<unsigned>((rows * 32 + threads - 1) / threads);
    att3::TimedLaunch timed(att3::K_SG_REDUCE, st);
    sgpack::sg_delta_kernel<D><<<blocks, threads, 0, st>>>(static_cast<const __nv_bfloat16*>(dY),
                                                           static_cast<const __nv_bfloat16*>(Y), delta, rows, t_ext.layout,
                                                           Hq, N);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_backward: delta launch");
    att3::count_launch(1);
    return ATT3_OK;
}

// The backward on the packed schedule: delta, dQ from the query-anchored kernel, then one key-side kernel per side.
static int pack_backward(int passes, bool kv_f32, const void* dY, const void* Q, const void* R, const void* S,
                         const void* Vr, const void* Vs, const void* Y, const float* m, const float* l,
                         const uint8_t* mask, void* dQ, void* dR, void* dS, void* dVr, void* dVs, int B, int Hq, int Hkv,
                         int N, int window, int q_begin, void* workspace, cudaStream_t st) {
    constexpr int D = 128;
    int* status = status_ptr();
    if (!status) return att3::set_error(ATT3_ERR_CUDA, "att3_sg_backward: status word not resolvable");
    const int W = pack_slots(window), QB = 128 / W;
    const int block_len = round_up8(bwd_block_len(B, Hkv, N));
    const int planes = sgring::bwd_planes(block_len);
    const int nblk = (N - q_begin + block_len - 1) / block_len;
    const size_t plane = static_cast<size_t>(B) * Hkv * N * D;
    float* part_K = static_cast<float*>(workspace);
    float* part_V = part_K + static_cast<size_t>(planes) * plane;
    // delta sits behind the planes the workspace was sized for (which may be more than this launch uses)
    float* delta = part_K + static_cast<size_t>(2 * sgring::bwd_planes(bwd_block_len(B, Hkv, N))) * plane;
    if (int rc = launch_delta<D>(dY, Y, delta, B, Hq, N, st)) return rc;
    int rc = ATT3_OK;
    sgpack::KvParams p{};
    p.Q = static_cast<const __nv_bfloat16*>(Q);
    p.dY = static_cast<const __nv_bfloat16*>(dY);
    p.m = m; p.l = l; p.delta = delta;
    p.mask = mask;
    p.mask_words = t_ext.mask_words;
    p.bnhd = t_ext.layout;
    p.part_K = part_K; p.part_V = part_V;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.N = N; p.window = window; p.q_begin = q_begin;
    p.block_len = block_len; p.planes = planes;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = status;
    sgring::BwdParams rp{};        // what launch_reduce reads
    rp.part_K = part_K; rp.part_V = part_V; rp.B = B; rp.Hkv = Hkv; rp.N = N; rp.q_begin = q_begin;
    rp.block_len = block_len; rp.planes = planes;
    auto kv_pass = [&](const void* ka, const void* va, const void* kb, const void* vb, void* dK, void* dV) {
        p.Ka = static_cast<const __nv_bfloat16*>(ka); p.Va = static_cast<const __nv_bfloat16*>(va);
        p.Kb = static_cast<const __nv_bfloat16*>(kb); p.Vb = static_cast<const __nv_bfloat16*>(vb);
        int r = W == 16 ? launch_pack_kv<16>(p, nblk, st) : W == 32 ? launch_pack_kv<32>(p, nblk, st) : launch_pack_kv<64>(p, nblk, st);
        if (r) return r;
        return launch_reduce(rp, nblk, D, dK, dV, st, kv_f32, QB - 1);
    };
    if (passes & 1) {
        if ((rc = run_pack_q(sgpack::PQ_DQ, Q, R, S, Vr, Vs, mask, nullptr, const_cast<float*>(m), const_cast<float*>(l), dY,
                             delta, dQ, B, Hq, Hkv, N, window, q_begin, status, st, "att3_sg_backward")))
            return rc;
        if ((rc = kv_pass(R, Vr, S, Vs, dS, dVs))) return rc;
    }
    if (passes & 2) rc = kv_pass(S, Vs, R, Vr, dR, dVr);
    return rc;
}

// passes: bit 0 = key side (S, Vs) with dQ, bit 1 = key side (R, Vr); both for a whole backward.
static int sg_backward_impl(int passes, bool kv_f32, const void* dY, const void* Q, const void* R, const void* S, const void* Vr,
                                const void* Vs, const void* Y, const float* m, const float* l,
                                const uint8_t* mask, void* dQ, void* dR, void* dS, void* dVr, void* dVs, int B,
                                int Hq, int Hkv, int N, int D, int window, int q_begin, void* workspace,
                                size_t workspace_bytes, void* stream) {
    if (int rc = check_shapes("att3_sg_backward", B, Hq, Hkv, N, D, window, q_begin)) return rc;
    if (!dY || !Q || !R || !S || !Vr || !Vs || !Y || !m || !l)
        return att3::set_error(ATT3_ERR_INVALID, "att3_sg_backward: null tensor pointer");
    if (((passes & 1) && (!dQ || !dS || !dVs)) || ((passes & 2) && (!dR || !dVr)))
        return att3::set_error(ATT3_ERR_INVALID, "att3_sg_backward: null gradient pointer");
    if (!att3::require_sm100("att3_sg_backward")) return ATT3_ERR_UNSUPPORTED;
    if (window == 0 && Hkv != Hq)
        return att3::set_error(ATT3_ERR_UNSUPPORTED, "att3_sg_backward: shared KV heads need a window (1..128)");
    if (window == 0 && q_begin != 0) return att3::set_error(ATT3_ERR_INVALID, "att3_sg_backward: q_begin needs a window");
    const size_t need = att3_sg_backward_workspace_bytes(B, Hq, Hkv, N, D, window);
    if (!workspace || workspace_bytes < need)
        return att3::set_error(ATT3_ERR_WORKSPACE, "att3_sg_backward: workspace of %zu bytes required, got %zu", need,
                               workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 16 != 0)
        return att3::set_error(ATT3_ERR_WORKSPACE, "att3_sg_backward: workspace must be 16-byte aligned");

    if (window == 0 && kv_f32)
        return att3::set_error(ATT3_ERR_UNSUPPORTED, "att3_sg_backward_kv32: only the windowed path (window 1..128) is offered");
    if (window == 0) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        const size_t plane = static_cast<size_t>(B) * Hq * N * D;
        const int nt = att3::dense_tiles(N, 0);
        float* ws = static_cast<float*>(workspace);
        float *gQ = ws, *gR = ws + plane, *gS = ws + 2 * plane, *gVr = ws + 3 * plane, *gVs = ws + 4 * plane,
              *part = ws + 5 * plane, *chunk_scratch = part + static_cast<size_t>(nt) * plane;
        cudaMemsetAsync(ws, 0, (5 + static_cast<size_t>(nt)) * plane * sizeof(float), st);
        int rc = att3::dense_gather_backward_side(Q, dY, Y, m, l, R, Vr, S, Vs, mask, gS, gVs, part, B, Hq, N, D, 0, st,
                                                  chunk_scratch);
        if (rc) return rc;
        if ((rc = att3::add_planes(part, nt, plane, gQ, st))) return rc;
        if ((rc = att3::dense_gather_backward_side(Q, dY, Y, m, l, S, Vs, R, Vr, mask, gR, gVr, nullptr, B, Hq, N, D, 0, st,
                                                   chunk_scratch)))
            return rc;
        att3::count_launch(1, 3);
        void* outs[5] = {dQ, dR, dS, dVr, dVs};
        const float* srcs[5] = {gQ, gR, gS, gVr, gVs};
        for (int k = 0; k < 5; ++k)
            if ((rc = att3::plane_to_bf16(srcs[k], outs[k], plane, st))) return rc;
        return ATT3_OK;
    }
    if (pack_eligible(Hq, Hkv, D, window, q_begin))
        return pack_backward(passes, kv_f32, dY, Q, R, S, Vr, Vs, Y, m, l, mask, dQ, dR, dS, dVr, dVs, B, Hq, Hkv, N, window,
                             q_begin, workspace, static_cast<cudaStream_t>(stream));
    sgring::BwdParams p;
    p.Q = static_cast<const __nv_bfloat16*>(Q);
    p.dY = static_cast<const __nv_bfloat16*>(dY);
    p.Y = static_cast<const __nv_bfloat16*>(Y);
    p.m = m; p.l = l;
    p.mask = mask;
    p.mask_words = t_ext.mask_words;
    p.bnhd = t_ext.layout;
    p.precise = t_ext.precise;
    p.dQ = static_cast<__nv_bfloat16*>(dQ);
    p.part_K = static_cast<float*>(workspace);
    p.block_len = bwd_block_len(B, Hkv, N);
    const int nblk = (N - q_begin + p.block_len - 1) / p.block_len;
    p.planes = sgring::bwd_planes(p.block_len);
    p.part_V = p.part_K + static_cast<size_t>(p.planes) * B * Hkv * N * D;
    // delta sits behind the partial planes; each call computes it (a call may be one key side of two)
    float* delta = p.part_K + static_cast<size_t>(2 * p.planes) * B * Hkv * N * D;
    p.delta = delta;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.N = N; p.window = window; p.q_begin = q_begin;
    p.scale = 1.0f / sqrtf(static_cast<float>(D));
    p.status = status_ptr();
    if (!p.status) return att3::set_error(ATT3_ERR_CUDA, "att3_sg_backward: status word not resolvable");
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    int rc = D == 64 ? launch_delta<64>(dY, Y, delta, B, Hq, N, st) : launch_delta<128>(dY, Y, delta, B, Hq, N, st);
    if (rc) return rc;
    if (passes & 1) {
        // Pass 1: own side (S, Vs) -> dS, dVs, and dQ.
        p.window = ext_window_s(window);
        p.window_oth = window;
        p.Ka = static_cast<const __nv_bfloat16*>(R);
        p.Va = static_cast<const __nv_bfloat16*>(Vr);
        p.Kb = static_cast<const __nv_bfloat16*>(S);
        p.Vb = static_cast<const __nv_bfloat16*>(Vs);
        rc = D == 64 ? launch_ring_bwd<64, true>(p, nblk, st) : launch_ring_bwd<128, true>(p, nblk, st);
        if (rc) return rc;
        if ((rc = launch_reduce(p, nblk, D, dS, dVs, st, kv_f32))) return rc;
    }
    if (!(passes & 2)) return ATT3_OK;
    // Pass 2: sides exchanged -> dR, dVr.
    p.window = window;
    p.window_oth = ext_window_s(window);
    p.Ka = static_cast<const __nv_bfloat16*>(S);
    p.Va = static_cast<const __nv_bfloat16*>(Vs);
    p.Kb = static_cast<const __nv_bfloat16*>(R);
    p.Vb = static_cast<const __nv_bfloat16*>(Vr);
    rc = D == 64 ? launch_ring_bwd<64, false>(p, nblk, st) : launch_ring_bwd<128, false>(p, nblk, st);
    if (rc) return rc;
    return launch_reduce(p, nblk, D, dR, dVr, st, kv_f32);
}

extern "C" int att3_sg_backward(const void* dY, const void* Q, const void* R, const void* S, const void* Vr,
                                const void* Vs, const void* Y, const float* m, const float* l,
                                const uint8_t* mask, void* dQ, void* dR, void* dS, void* dVr, void* dVs, int B,
                                int Hq, int Hkv, int N, int D, int window, int q_begin, void* workspace,
                                size_t workspace_bytes, void* stream) {
    return sg_backward_impl(3, false, dY, Q, R, S, Vr, Vs, Y, m, l, mask, dQ, dR, dS, dVr, dVs, B, Hq, Hkv, N, D, window,
                            q_begin, workspace, workspace_bytes, stream);
}

// The same backward with the four key-side gradients left in FP32 ([B,Hkv,N,D] floats): for a rank that holds
// only part of the query heads of a KV head, whose sums are partials to be added across ranks before rounding.
extern "C" int att3_sg_backward_kv32(const void* dY, const void* Q, const void* R, const void* S, const void* Vr,
                                     const void* Vs, const void* Y, const float* m, const float* l,
                                     const uint8_t* mask, void* dQ, float* dR, float* dS, float* dVr, float* dVs,
                                     int B, int Hq, int Hkv, int N, int D, int window, int q_begin, void* workspace,
                                     size_t workspace_bytes, void* stream) {
    return sg_backward_impl(3, true, dY, Q, R, S, Vr, Vs, Y, m, l, mask, dQ, dR, dS, dVr, dVs, B, Hq, Hkv, N, D, window,
                            q_begin, workspace, workspace_bytes, stream);
}

// One key side of att3_sg_backward_kv32 at a time, so that a caller can start exchanging the first side's
// sums (dS, dVs) with other processes while the second side is computed.
extern "C" int att3_sg_backward_kv32_side(int side, const void* dY, const void* Q, const void* R, const void* S,
                                          const void* Vr, const void* Vs, const void* Y, const float* m,
                                          const float* l, const uint8_t* mask, void* dQ, float* dR, float* dS,
                                          float* dVr, float* dVs, int B, int Hq, int Hkv, int N, int D, int window,
                                          int q_begin, void* workspace, size_t workspace_bytes, void* stream) {
    if (side != 0 && side != 1)
        return att3::set_error(ATT3_ERR_INVALID, "att3_sg_backward_kv32_side: side must be 0 (S, Vs, dQ) or 1 (R, Vr)");
    return sg_backward_impl(side == 0 ? 1 : 2, true, dY, Q, R, S, Vr, Vs, Y, m, l, mask, dQ, dR, dS, dVr, dVs, B, Hq, Hkv,
                            N, D, window, q_begin, workspace, workspace_bytes, stream);
}


// ---------------------------------------------------------------------------
// Extended calls: asymmetric windows, packed masks
// ---------------------------------------------------------------------------

static int check_ext(const char* who, const att3_sg_ext* ext, int window, const uint8_t* mask) {
    if (!ext) return ATT3_OK;
    if (ext->window_s < 0 || ext->window_s > sgring::RING)
        return att3::set_error(ATT3_ERR_INVALID, "%s: window_s must be in [0,128], got %d", who, ext->window_s);
    if ((ext->window_s > 0 || ext->mask_words) && window == 0)
        return att3::set_error(ATT3_ERR_UNSUPPORTED, "%s: window_s and packed masks need the windowed path (window 1..128)", who);
    if (ext->mask_words && mask)
        return att3::set_error(ATT3_ERR_INVALID, "%s: pass the mask either as bytes or as packed words, not both", who);
    if (ext->mask_words && reinterpret_cast<uintptr_t>(ext->mask_words) % 4 != 0)
        return att3::set_error(ATT3_ERR_INVALID, "%s: mask_words must be 4-byte aligned", who);
    if (ext->layout != 0 && ext->layout != 1)
        return att3::set_error(ATT3_ERR_INVALID, "%s: layout must be 0 ([B,H,N,D]) or 1 ([B,N,H,D]), got %d", who, ext->layout);
    if (ext->precise && window == 0)
        return att3::set_error(ATT3_ERR_UNSUPPORTED, "%s: the compensated products need the windowed path (window 1..128)", who);
    if ((ext->layout || ext->Y_act) && window == 0)
        return att3::set_error(ATT3_ERR_UNSUPPORTED, "%s: the [B,N,H,D] layout and the activated output need the windowed path (window 1..128)", who);
    return ATT3_OK;
}

struct ExtScope {       // sets the calling thread's extension state for the duration of one call
    explicit ExtScope(const att3_sg_ext* ext) { if (ext) t_ext = SgExt{ext->window_s, ext->mask_words, ext->layout, ext->Y_act, ext->precise}; }
    ~ExtScope() { t_ext = SgExt{0, nullptr, 0, nullptr, 0}; }
};

extern "C" int att3_sg_forward_ext(const void* Q, const void* R, const void* S, const void* Vr, const void* Vs,
                                   const uint8_t* mask, void* Y, float* m, float* l, int B, int Hq, int Hkv, int N,
                                   int D, int window, int q_begin, void* stream, const att3_sg_ext* ext) {
    if (int rc = check_ext("att3_sg_forward_ext", ext, window, mask)) return rc;
    ExtScope scope(ext);
    return att3_sg_forward(Q, R, S, Vr, Vs, mask, Y, m, l, B, Hq, Hkv, N, D, window, q_begin, stream);
}

extern "C" int att3_sg_backward_ext(const void* dY, const void* Q, const void* R, const void* S, const void* Vr,
                                    const void* Vs, const void* Y, const float* m, const float* l,
                                    const uint8_t* mask, void* dQ, void* dR, void* dS, void* dVr, void* dVs, int B,
                                    int Hq, int Hkv, int N, int D, int window, int q_begin, void* workspace,
                                    size_t workspace_bytes, void* stream, const att3_sg_ext* ext) {
    if (int rc = check_ext("att3_sg_backward_ext", ext, window, mask)) return rc;
    ExtScope scope(ext);
    return att3_sg_backward(dY, Q, R, S, Vr, Vs, Y, m, l, mask, dQ, dR, dS, dVr, dVs, B, Hq, Hkv, N, D, window, q_begin,
                            workspace, workspace_bytes, stream);
}

// Packs a byte mask into words and counts each query's visible keys inside its causal window, saturated at 2
// (0 dead, 1 a single key: exact-zero score gradients, 2 anything more): the metadata pass of the reference
// (att3_mask_metadata::prepare, cuda/shared_kv/shared_mask_metadata.cuh:8-31).  One warp per query row.
__global__ void pack_mask_kernel(const uint8_t* mask, uint32_t* words, uint8_t* support, int B, int N, int window) {
    const size_t row = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= static_cast<size_t>(B) * N) return;
    const int i = static_cast<int>(row % N), NW = (N + 31) / 32;
    const uint8_t* src = mask + row * N;
    int count = 0;
    for (int c = 0; c < NW; ++c) {
        const int key = c * 32 + lane;
        bool v = key < N && src[key] != 0;
        if (window > 0) v = v && key <= i && key > i - window;
        const uint32_t w = __ballot_sync(0xFFFFFFFFu, v);
        if (lane == 0) words[row * NW + c] = w;
        count += __popc(w);
    }
    if (support && lane == 0) support[row] = static_cast<uint8_t>(count > 2 ? 2 : count);
}

extern "C" int att3_sg_pack_mask(const uint8_t* mask, uint32_t* words, uint8_t* support, int B, int N, int window,
                                 void* stream) {
    if (!mask || !words || B <= 0 || N <= 0 || window < 0)
        return att3::set_error(ATT3_ERR_INVALID, "att3_sg_pack_mask: bad argument");
    const size_t rows = static_cast<size_t>(B) * N;
    const int threads = 256;
    pack_mask_kernel<<<static_cast<unsigned>((rows * 32 + threads - 1) / threads), threads, 0,
                       static_cast<cudaStream_t>(stream)>>>(mask, words, support, B, N, window);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ATT3_OK : att3::set_cuda_error(e, "att3_sg_pack_mask: launch");
}

// ---------------------------------------------------------------------------
// Backward for callers that cannot allocate
// ---------------------------------------------------------------------------
//
// Some hosts of this library have no way to hand the backward a scratch buffer:
// a plugin running inside a framework's stream-ordered or graph-private memory
// pool where cudaMalloc is forbidden, a real-time inference/training loop that
// pre-plans all device memory and treats any allocator call as a fault, or a
// sandboxed worker whose CUDA allocation entry points are not reachable at all.
// For them the FP32 key-gradient partials of the windowed backward live in a
// fixed array that is part of the library image.  Every GPU that loads the
// library holds these ATT3_STATIC_SCRATCH_BYTES until the process exits.
//
// The array's name is only a host-side handle: its device address is looked up
// once per device, with that device current, by cudaGetSymbolAddress, and that
// address is what the kernels receive.
constexpr size_t ATT3_STATIC_SCRATCH_BYTES = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[ATT3_STATIC_SCRATCH_BYTES];

extern "C" size_t att3_sg_backward_static_max_bytes(void) { return ATT3_STATIC_SCRATCH_BYTES; }

extern "C" int att3_sg_backward_static(const void* dY, const void* Q, const void* R, const void* S, const void* Vr,
                                       const void* Vs, const void* Y, const float* m, const float* l,
                                       const uint8_t* mask, void* dQ, void* dR, void* dS, void* dVr, void* dVs,
                                       int B, int Hq, int Hkv, int N, int D, int window, int q_begin, void* stream) {
    if (window < 1 || window > sgring::RING)
        return att3::set_error(ATT3_ERR_INVALID,
                               "att3_sg_backward_static: only the windowed path (window 1..128) is offered, got %d",
                               window);
    if (int rc = check_shapes("att3_sg_backward_static", B, Hq, Hkv, N, D, window, q_begin)) return rc;
    const size_t need = att3_sg_backward_workspace_bytes(B, Hq, Hkv, N, D, window);
    if (need > ATT3_STATIC_SCRATCH_BYTES)
        return att3::set_error(ATT3_ERR_WORKSPACE,
                               "att3_sg_backward_static: these sizes need %zu bytes of scratch "
                               "(att3_sg_backward_workspace_bytes), the built-in array holds %zu; use "
                               "att3_sg_backward with a workspace",
                               need, ATT3_STATIC_SCRATCH_BYTES);
    // Device address of the array, resolved on the first call per device (keep that call outside
    // any stream capture) and cached afterwards.
    constexpr int kMaxDevices = 64;
    static void* cached[kMaxDevices] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_sg_backward_static: cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices)
        return att3::set_error(ATT3_ERR_UNSUPPORTED, "att3_sg_backward_static: device ordinal %d out of range", dev);
    void* ptr = cached[dev];
    if (!ptr) {
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return att3::set_cuda_error(e, "att3_sg_backward_static: cudaGetSymbolAddress(scratch)");
        cached[dev] = ptr;
    }
    // Nothing in the scratch has to start at zero: every partial row the reduction reads is
    // written by exactly one CTA of the same call first.  The array is shared by all calls,
    // so two calls whose kernels may overlap on the device (different streams) race on it.
    return att3_sg_backward(dY, Q, R, S, Vr, Vs, Y, m, l, mask, dQ, dR, dS, dVr, dVs, B, Hq, Hkv, N, D, window,
                            q_begin, ptr, ATT3_STATIC_SCRATCH_BYTES, stream);
}
