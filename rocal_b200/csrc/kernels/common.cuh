// Shared device helpers and host-side launch bookkeeping of the sm_100a kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rb200_kernels.h"

namespace rb200 {

// ---- host-side bookkeeping (defined in runtime.cu) -------------------------------------
void set_error(const char* fmt, ...);
void count_launch();
int check_cuda(cudaError_t e, const char* what);
// Device address of the library-wide status word of the current device (runtime.cu); nullptr if the query failed.
int* default_status_word();
// Reads and clears that word: 0 / 1, or -1 when the copy failed.
int read_default_status_word();
constexpr unsigned long long kDefaultWaitCycles = 2000000000ull;   // about a second of SM clock

#define RB200_CHECK_LAUNCH(what)                                       \
    do {                                                               \
        ::rb200::count_launch();                                       \
        int _rc = ::rb200::check_cuda(cudaGetLastError(), what);       \
        if (_rc) return _rc;                                           \
    } while (0)

static inline uint64_t out_elem_size(int out_dtype) { return out_dtype == RB200_FP32 ? 4 : out_dtype == RB200_FP16 ? 2 : 1; }

// ---- status word and the bounds-checking build ------------------------------------------------
// A kernel reports trouble by writing its status word and returning normally: 1 = a bounded wait ran out,
// 2 = (bounds-checking build only) a read would have left the source arena and was not made. The larger value stays.
constexpr int kStatusWaitRanOut = 1, kStatusOutOfBounds = 2;
__device__ __forceinline__ void raise_status(int* status, int value = kStatusWaitRanOut) {
    volatile int* p = reinterpret_cast<volatile int*>(status);
    if (*p < value) *p = value;
    __threadfence_system();
}

#ifdef RB200_DEBUG_BOUNDS
constexpr bool kCheckBounds = true;
#else
constexpr bool kCheckBounds = false;
#endif

// The addresses a launch may read: the source arena widened to whole 16-byte granules (the staging copies fetch the
// granules that enclose a row span; device and pinned allocations are far coarser than 16 bytes). hi == nullptr: the
// caller gave no size, nothing is checked. The checks below compile to nothing outside the bounds-checking build.
struct ArenaBounds {
    const uint8_t* lo;
    const uint8_t* hi;
};
static inline ArenaBounds arena_bounds(const uint8_t* arena, uint64_t bytes) {
    ArenaBounds b = {nullptr, nullptr};
    if (kCheckBounds && bytes) {
        b.lo = reinterpret_cast<const uint8_t*>((uintptr_t)arena & ~(uintptr_t)15);
        b.hi = reinterpret_cast<const uint8_t*>(((uintptr_t)arena + bytes + 15) & ~(uintptr_t)15);
    }
    return b;
}
// One contiguous read [p, p + bytes).
__device__ __forceinline__ bool span_in_bounds(const ArenaBounds& b, const void* p, size_t bytes, int* status) {
    if (!kCheckBounds || b.hi == nullptr) return true;
    const uint8_t* q = reinterpret_cast<const uint8_t*>(p);
    if (q >= b.lo && q <= b.hi && bytes <= (size_t)(b.hi - q)) return true;
    raise_status(status, kStatusOutOfBounds);
    return false;
}
// The w x h pixel rectangle at (x, y) of a 3-byte-per-pixel image, each row span widened to its 16-byte granules.
__device__ __forceinline__ bool rect_in_bounds(const ArenaBounds& b, const uint8_t* img, uint32_t stride, int x, int y, int w, int h,
                                               int* status) {
    if (!kCheckBounds || b.hi == nullptr) return true;
    bool ok = x >= 0 && y >= 0 && w > 0 && h > 0;
    if (ok) {
        const uintptr_t first = ((uintptr_t)img + (size_t)y * stride + (size_t)x * 3) & ~(uintptr_t)15;
        const uintptr_t end = ((uintptr_t)img + (size_t)(y + h - 1) * stride + (size_t)(x + w) * 3 + 15) & ~(uintptr_t)15;
        ok = first >= (uintptr_t)b.lo && end <= (uintptr_t)b.hi && first < end;
    }
    if (!ok) raise_status(status, kStatusOutOfBounds);
    return ok;
}

// ---- programmatic dependent launch ---------------------------------------------------------
// Kernels of this library that follow one another in a stream overlap their ramp-up with the predecessor's
// tail: a launch made with launch_overlapped() may be scheduled as soon as every CTA of the preceding kernel has
// started (each calls pdl_launch_dependents() on entry), and its CTAs park in pdl_wait() until that kernel has
// completed and its writes are visible. Everything that reads or writes global memory comes after pdl_wait(), so
// the result is that of a plain in-order launch; what is saved is the launch gap and the block-scheduling ramp
// of small batches. Behind anything that is not a kernel (a copy, an event wait) the launch is an ordinary one.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                            Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// ---- arithmetic with one rounding per operation ------------------------------------------
// The CPU checker is built without contraction, so every product that feeds a sum is written
// with the non-fusing intrinsics; fused operations are spelled fmaf().
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float div_rn(float a, float b) { return __fdiv_rn(a, b); }

// Round to nearest even for |v| < 2^22 (two adds instead of a conversion round trip).
__device__ __forceinline__ float rint_small(float v) {
    return __fsub_rn(__fadd_rn(v, 12582912.0f), 12582912.0f);
}

// Round to nearest even and saturate to [0,255], result kept as float.
__device__ __forceinline__ float sat_round_u8f(float v) {
    // fminf/fmaxf return the non-NaN operand, so NaN maps to 0 like the checker's !(r > 0).
    float c = fminf(fmaxf(v, 0.0f), 255.0f);
    return rint_small(c);
}

template <typename T>
struct OutConv;
template <>
struct OutConv<float> {
    static __device__ __forceinline__ float cvt(float v) { return v; }
};
template <>
struct OutConv<__half> {
    static __device__ __forceinline__ __half cvt(float v) { return __float2half_rn(v); }
};
template <>
struct OutConv<uint8_t> {
    static __device__ __forceinline__ uint8_t cvt(float v) { return (uint8_t)sat_round_u8f(v); }
};

// Four bytes starting at an arbitrary byte offset of a 4-byte-aligned shared-memory row.
__device__ __forceinline__ uint32_t lds_unaligned32(const uint8_t* row, int byte_off) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(row + (byte_off & ~3));
    return __funnelshift_r(w[0], w[1], (byte_off & 3) * 8);
}

__device__ __forceinline__ float byte_to_float(uint32_t w, int idx) {
    return (float)((w >> (8 * idx)) & 0xFFu);
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    uint32_t s = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

// ---- packed f32x2 arithmetic (sm_100): both lanes rounded independently, round-to-nearest ----
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long ra = *reinterpret_cast<unsigned long long*>(&a);
    unsigned long long rb = *reinterpret_cast<unsigned long long*>(&b);
    unsigned long long rc = *reinterpret_cast<unsigned long long*>(&c), rd;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    return *reinterpret_cast<float2*>(&rd);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    unsigned long long ra = *reinterpret_cast<unsigned long long*>(&a);
    unsigned long long rb = *reinterpret_cast<unsigned long long*>(&b), rd;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    return *reinterpret_cast<float2*>(&rd);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long ra = *reinterpret_cast<unsigned long long*>(&a);
    unsigned long long rb = *reinterpret_cast<unsigned long long*>(&b), rd;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    return *reinterpret_cast<float2*>(&rd);
}

}  // namespace rb200
