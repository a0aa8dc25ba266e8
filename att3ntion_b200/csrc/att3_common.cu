// Host-side plumbing behind the C ABI: thread-local error text, device checks,
// launch counters, and the window -> tile-range / mask-packing helpers that need
// no GPU.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "att3_abi_internal.h"

namespace att3 {

static thread_local char g_err[512] = "";
static std::atomic<unsigned long long> g_launches[4];

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int set_cuda_error(cudaError_t e, const char* where) {
    return set_error(ATT3_ERR_CUDA, "%s: %s", where, cudaGetErrorString(e));
}

bool require_sm100(const char* who) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        set_error(ATT3_ERR_UNSUPPORTED, "%s: tensor-core path unavailable, no CUDA device (%s)", who,
                  cudaGetErrorString(e));
        return false;
    }
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (major != 10) {
        set_error(ATT3_ERR_UNSUPPORTED,
                  "%s: tensor-core path unavailable on this device (built for sm_100a, device is sm_%d0)", who,
                  major);
        return false;
    }
    return true;
}

int sm_count() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
        cached_dev = dev;
    }
    return cached > 0 ? cached : 148;
}

void count_launch(int which, int n) {
    if (which >= 0 && which < 4) g_launches[which] += n;
}

// ---- optional per-kernel timing ------------------------------------------------
struct TimingRec { int id; cudaEvent_t a, b; };
static std::mutex g_time_mu;
static std::vector<TimingRec> g_time_recs;
static std::atomic<int> g_time_on{0};

TimedLaunch::TimedLaunch(int kernel_id, cudaStream_t stream) : id_(kernel_id), stream_(stream) {
    if (!g_time_on.load(std::memory_order_relaxed)) return;
    if (cudaEventCreate(&start_) != cudaSuccess) { start_ = nullptr; return; }
    cudaEventRecord(start_, stream_);
}

TimedLaunch::~TimedLaunch() {
    if (!start_) return;
    cudaEvent_t stop = nullptr;
    if (cudaEventCreate(&stop) != cudaSuccess) { cudaEventDestroy(start_); return; }
    cudaEventRecord(stop, stream_);
    std::lock_guard<std::mutex> lk(g_time_mu);
    g_time_recs.push_back({id_, start_, stop});
}

int make_row_tensor_map(CUtensorMap* out, const void* base, size_t rows, int cols, const char* who, int box_rows,
                        int pitch_cols) {
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return reinterpret_cast<EncodeFn>(fn);
    }();
    if (!encode) return set_error(ATT3_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available from this driver", who);
    if (cols <= 0 || cols > 256 || (cols * 2) % 16 != 0 || reinterpret_cast<uintptr_t>(base) % 16 != 0)
        return set_error(ATT3_ERR_INVALID, "%s: row tensor map needs 16-byte aligned rows of at most 256 BF16", who);
    if (pitch_cols <= 0) pitch_cols = cols;
    if (pitch_cols % cols != 0) return set_error(ATT3_ERR_INVALID, "%s: row pitch must be a multiple of the row length", who);
    // the matrix is [rows, pitch_cols]; a box is `box_rows` rows of `cols` columns starting at a multiple of `cols`
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(pitch_cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_cols) * 2};       // bytes between rows
    if (box_rows < 1 || box_rows > 256) return set_error(ATT3_ERR_INVALID, "%s: tensor map box of %d rows", who, box_rows);
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(cols), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(ATT3_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed (CUresult %d)", who, int(r));
    return ATT3_OK;
}

int make_head_tensor_map(CUtensorMap* out, const void* base, int B, int H, int N, int D, int bnhd, int box_rows,
                         const char* who) {
    if (bnhd) return make_row_tensor_map(out, base, static_cast<size_t>(B) * N, D, who, box_rows, H * D);
    return make_row_tensor_map(out, base, static_cast<size_t>(B) * H * N, D, who, box_rows, D);
}

}  // namespace att3

extern "C" int att3_timing_enable(int on) { return att3::g_time_on.exchange(on ? 1 : 0); }

extern "C" int att3_timing_read(int kernel_id, double* total_ms, unsigned long long* launches) {
    if (kernel_id < 0 || kernel_id >= att3::K_COUNT || !total_ms || !launches)
        return att3::set_error(ATT3_ERR_INVALID, "att3_timing_read: bad argument");
    double sum = 0.0;
    unsigned long long n = 0;
    std::lock_guard<std::mutex> lk(att3::g_time_mu);
    auto& recs = att3::g_time_recs;
    for (size_t i = 0; i < recs.size();) {
        if (recs[i].id != kernel_id) { ++i; continue; }
        cudaError_t e = cudaEventSynchronize(recs[i].b);
        float ms = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, recs[i].a, recs[i].b);
        cudaEventDestroy(recs[i].a);
        cudaEventDestroy(recs[i].b);
        recs.erase(recs.begin() + i);
        if (e != cudaSuccess) return att3::set_cuda_error(e, "att3_timing_read");
        sum += ms;
        ++n;
    }
    *total_ms = sum;
    *launches = n;
    return ATT3_OK;
}

extern "C" const char* att3_last_error(void) { return att3::g_err; }

extern "C" int att3_abi_version(void) { return 2; }

extern "C" unsigned long long att3_launch_count(int which) {
    return (which >= 0 && which < 4) ? att3::g_launches[which].load() : 0ull;
}

// Rows and columns a windowed single-gather work item has to visit.  The
// interval starts on the first visible key rather than on a tile boundary, ends
// are exclusive, and the column end is rounded up to a multiple of bk counted
// from the start, so padding never widens the set of visited real keys.
//   side 0 (query is anchor a): rows and cols are both (a - w, a].
//   side 1 (a is a key, queries are rows): rows [a, a + w); a row block at j0
//          needs cols (j0 - w, min(j0 + bj, a + w, N)).
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

static void row_range(int side, int a, int N, int w, int* lo, int* hi) {
    if (w <= 0) { *lo = 0; *hi = N; return; }
    int l = side == 0 ? a - w + 1 : a;
    int h = side == 0 ? a + 1 : a + w;
    *lo = l < 0 ? 0 : l;
    *hi = h > N ? N : h;
}

static void col_range(int side, int a, int j0, int bj, int N, int w, int bk, int* lo, int* hi) {
    if (w <= 0) { *lo = 0; *hi = ceil_div(N, bk) * bk; return; }
    int l = side == 0 ? a - w + 1 : j0 - w + 1;
    int h = side == 0 ? a + 1 : j0 + bj;
    if (side == 1 && h > a + w) h = a + w;
    if (l < 0) l = 0;
    if (h > N) h = N;
    *lo = l;
    *hi = l + ceil_div(h - l, bk) * bk;
}

extern "C" int att3_sg_tile_ranges(int N, int window, int a, int side, int bj, int bk, int* out, int max_out) {
    if (N <= 0 || a < 0 || a >= N || (side != 0 && side != 1) || bj <= 0 || bk <= 0 || (max_out > 0 && !out))
        return -1;
    int lo, hi, n = 0;
    row_range(side, a, N, window, &lo, &hi);
    for (int j0 = lo; j0 < hi; j0 += bj, ++n) {
        if (n < max_out) {
            int kl, kh;
            col_range(side, a, j0, bj, N, window, bk, &kl, &kh);
            out[3 * n] = j0;
            out[3 * n + 1] = kl;
            out[3 * n + 2] = kh;
        }
    }
    return n;
}

extern "C" uint32_t att3_pack_mask32(const uint8_t* row, int lim) {
    uint32_t bits = 0;
    if (lim > 32) lim = 32;
    int t = 0;
    // Byte loads until the pointer is 4-byte aligned, then whole words that lie
    // entirely inside [row, row + lim), then the tail.
    for (; t < lim && ((reinterpret_cast<uintptr_t>(row + t)) & 3u); ++t)
        if (row[t]) bits |= 1u << t;
    for (; t + 4 <= lim; t += 4) {
        uint32_t w;
        memcpy(&w, row + t, 4);
        for (int b = 0; b < 4; ++b)
            if ((w >> (8 * b)) & 0xFFu) bits |= 1u << (t + b);
    }
    for (; t < lim; ++t)
        if (row[t]) bits |= 1u << t;
    return bits;
}
