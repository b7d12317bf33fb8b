// Normalize: out = scale * (x - mean) / stddev + shift on uint8 HWC images, statistics given or computed over
// a chosen set of axes; and Transpose (axis permutation of uint8 HWC images).
//
// Computed statistics go through scratch memory: per sample and statistic index one slot of two 64-bit integers
// (sum of x, sum of x^2). Integer sums are exact and independent of the order in which the atomics land, so the
// result is deterministic; a one-block-per-sample finishing kernel turns each slot into (mean, scale / stddev) as two
// floats, evaluated in double, and the element-wise pass reads those.
//
//   sums      grid = (row tiles, samples), 192 threads: a thread owns byte columns j, j + 192, ... of the sample's
//             rows (192 = 64 pixels, so a thread's channel never changes) and walks down the tile's rows; column-wise
//             statistics leave through one atomic pair per thread and column, per-channel / per-image ones through
//             shared-memory atomics and six global ones per CTA; row-wise statistics take a warp per row (30 lanes =
//             10 pixels, lanes 30 and 31 idle) and need no global atomics: a row belongs to one warp.
//   finish    grid = samples.
//   apply     grid = (row tiles, samples), 256 threads, one output element per thread and step: consecutive threads
//             read consecutive bytes and write consecutive floats.
// The source rows are read with plain byte loads: the kernels are bound by the float output (4 bytes out per byte
// in), not by the load instructions.
#include "common.cuh"

namespace rb200 {

struct StatSlot {
    unsigned long long s1, s2;      // after the finishing kernel: float mean, float mult in the first 8 bytes
};

struct NormLaunch {
    void* out;
    int out_w, out_h, fp16;
    int mask, slots;                // slots per sample (0: nothing is computed)
    int compute_mean, compute_stddev, fill_padding;
    float mean[3], stddev[3], scale, shift;
    StatSlot* stats;
    int th;                         // rows per tile
    int* status;                    // bounds-checking build: written with 2 when a sample's window leaves the arena
    ArenaBounds bounds;             // bounds-checking build: the addresses the launch may read
};

// Slot index of element (y, x, c) under a mask; the slot count is stat_slots().
__device__ __forceinline__ int stat_index(int mask, int y, int x, int c, int w) {
    switch (mask) {
        case 1: return x * 3 + c;   // reduce H          -> per (x, c)
        case 2: return y * 3 + c;   // reduce W          -> per (y, c)
        case 3: return c;           // reduce H, W       -> per channel
        case 4: return y * w + x;   // reduce C          -> per pixel
        case 5: return x;           // reduce H, C       -> per column
        case 6: return y;           // reduce W, C       -> per row
        default: return 0;          // 7: per image
    }
}

static int stat_slots(int mask, int w, int h) {
    switch (mask) {
        case 1: return 3 * w;
        case 2: return 3 * h;
        case 3: return 3;
        case 4: return w * h;
        case 5: return w;
        case 6: return h;
        case 7: return 1;
        default: return 0;
    }
}

__device__ __forceinline__ void slot_add(StatSlot* s, unsigned long long a, unsigned long long b) {
    atomicAdd(&s->s1, a);
    atomicAdd(&s->s2, b);
}

__global__ void __launch_bounds__(192) normalize_sums_kernel(const uint8_t* __restrict__ arena,
                                                              const rb200_pointwise_sample* __restrict__ samples,
                                                              const NormLaunch L) {
    __shared__ unsigned long long sh[6];
    const int n = blockIdx.y;
    const rb200_pointwise_sample s = samples[n];
    const int w = min(s.roi_w, L.out_w), h = min(s.roi_h, L.out_h);
    const int y0 = blockIdx.x * L.th, y1 = min(y0 + L.th, h);
    if (y0 >= h || w <= 0) return;
    if (!rect_in_bounds(L.bounds, arena + s.src_offset, s.src_stride, s.roi_x, s.roi_y, s.roi_w, s.roi_h, L.status)) return;
    const uint8_t* img = arena + s.src_offset + (size_t)s.roi_y * s.src_stride + (size_t)s.roi_x * 3;
    StatSlot* st = L.stats + (size_t)n * L.slots;
    const int rowbytes = 3 * w;
    const int mask = L.mask;
    if (mask == 2 || mask == 6 || mask == 4) {
        // row-wise (and per-pixel) statistics: one warp per row, lanes 0..29 stride over the row's bytes
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (int y = y0 + warp; y < y1; y += 6) {
            const uint8_t* row = img + (size_t)y * s.src_stride;
            if (mask == 4) {
                for (int x = lane; x < w; x += 32) {
                    const unsigned a = row[3 * x], b = row[3 * x + 1], c = row[3 * x + 2];
                    st[y * w + x].s1 = a + b + c;
                    st[y * w + x].s2 = a * a + b * b + c * c;
                }
                continue;
            }
            unsigned a1 = 0, a2 = 0;
            if (lane < 30)
                for (int j = lane; j < rowbytes; j += 30) {
                    const unsigned v = row[j];
                    a1 += v;
                    a2 += v * v;
                }
            // lanes of one channel are lane, lane + 3, ...: fold the ten of them (and for mask 6 all thirty)
            unsigned long long t1 = a1, t2 = a2;
            if (mask == 6) {
                for (int o = 16; o > 0; o >>= 1) {
                    t1 += __shfl_xor_sync(0xffffffffu, t1, o);
                    t2 += __shfl_xor_sync(0xffffffffu, t2, o);
                }
                if (lane == 0) { st[y].s1 = t1; st[y].s2 = t2; }
            } else {
                // channel sums: gather lanes c, c+3, ..., c+27 into lane c
                unsigned long long c1 = 0, c2 = 0;
                for (int k = 0; k < 10; k++) {
                    const unsigned long long o1 = __shfl_sync(0xffffffffu, t1, (lane % 3) + 3 * k);
                    const unsigned long long o2 = __shfl_sync(0xffffffffu, t2, (lane % 3) + 3 * k);
                    c1 += o1;
                    c2 += o2;
                }
                if (lane < 3) { st[y * 3 + lane].s1 = c1; st[y * 3 + lane].s2 = c2; }
            }
        }
        return;
    }
    // column-wise, per-channel and per-image statistics: a thread owns byte columns tid, tid + 192, ...
    if (threadIdx.x < 6) sh[threadIdx.x] = 0ull;
    __syncthreads();
    const int c = threadIdx.x % 3;
    unsigned long long p1 = 0, p2 = 0;
    for (int j = threadIdx.x; j < rowbytes; j += 192) {
        unsigned a1 = 0, a2 = 0;
        const uint8_t* p = img + (size_t)y0 * s.src_stride + j;
        for (int y = y0; y < y1; y++, p += s.src_stride) {
            const unsigned v = *p;
            a1 += v;
            a2 += v * v;
        }
        if (mask == 1) slot_add(&st[j], a1, a2);              // per (x, c): j = 3x + c
        else if (mask == 5) slot_add(&st[j / 3], a1, a2);     // per column
        else { p1 += a1; p2 += a2; }
    }
    if (mask == 3 || mask == 7) {
        atomicAdd(&sh[2 * c], p1);
        atomicAdd(&sh[2 * c + 1], p2);
        __syncthreads();
        if (mask == 3) {
            if (threadIdx.x < 3) slot_add(&st[threadIdx.x], sh[2 * threadIdx.x], sh[2 * threadIdx.x + 1]);
        } else if (threadIdx.x == 0) {
            slot_add(&st[0], sh[0] + sh[2] + sh[4], sh[1] + sh[3] + sh[5]);
        }
    }
}

// Number of values behind one statistic of a w x h x 3 window.
__device__ __forceinline__ double stat_count(int mask, int w, int h) {
    switch (mask) {
        case 1: return (double)h;
        case 2: return (double)w;
        case 3: return (double)w * h;
        case 4: return 3.0;
        case 5: return 3.0 * h;
        case 6: return 3.0 * w;
        default: return 3.0 * w * h;
    }
}

// Channel a slot belongs to when a given per-channel constant is needed beside a computed statistic (-1: the slot
// spans the channels, the constant of channel 0 is used).
__device__ __forceinline__ int slot_channel(int mask, int idx) {
    if (mask == 1 || mask == 2) return idx % 3;
    if (mask == 3) return idx;
    return -1;
}

__global__ void normalize_finish_kernel(const rb200_pointwise_sample* __restrict__ samples, const NormLaunch L) {
    const int n = blockIdx.x;
    const rb200_pointwise_sample s = samples[n];
    const int w = min(s.roi_w, L.out_w), h = min(s.roi_h, L.out_h);
    if (w <= 0 || h <= 0) return;
    const int mask = L.mask;
    int used = 0;
    switch (mask) {
        case 1: used = 3 * w; break;
        case 2: used = 3 * h; break;
        case 3: used = 3; break;
        case 4: used = w * h; break;
        case 5: used = w; break;
        case 6: used = h; break;
        default: used = 1;
    }
    const double cnt = stat_count(mask, w, h);
    StatSlot* st = L.stats + (size_t)n * L.slots;
    for (int i = threadIdx.x; i < used; i += blockDim.x) {
        const double s1 = (double)st[i].s1, s2 = (double)st[i].s2;
        const int ch = slot_channel(mask, i);
        float mean_f = L.compute_mean ? (float)(s1 / cnt) : L.mean[ch < 0 ? 0 : ch];
        float std_f;
        if (L.compute_stddev) {
            const double m = (double)mean_f;
            double var = (s2 - 2.0 * m * s1) / cnt + m * m;
            if (!(var > 0.0)) var = 0.0;
            std_f = (float)sqrt(var);
        } else {
            std_f = L.stddev[ch < 0 ? 0 : ch];
        }
        const float mult = std_f > 0.f ? __fdiv_rn(L.scale, std_f) : 0.f;
        float2 r = make_float2(mean_f, mult);
        *reinterpret_cast<float2*>(&st[i]) = r;
    }
}

template <typename OutT>
__global__ void __launch_bounds__(256) normalize_apply_kernel(const uint8_t* __restrict__ arena,
                                                               const rb200_pointwise_sample* __restrict__ samples,
                                                               const NormLaunch L) {
    const int n = blockIdx.y;
    const rb200_pointwise_sample s = samples[n];
    const int w = min(s.roi_w, L.out_w), h = min(s.roi_h, L.out_h);
    const int y0 = blockIdx.x * L.th;
    const int rows = min(L.th, L.out_h - y0);
    if (rows <= 0) return;
    if (w > 0 && h > 0 &&
        !rect_in_bounds(L.bounds, arena + s.src_offset, s.src_stride, s.roi_x, s.roi_y, s.roi_w, s.roi_h, L.status))
        return;
    const uint8_t* img = arena + s.src_offset + (size_t)s.roi_y * s.src_stride + (size_t)s.roi_x * 3;
    OutT* out = reinterpret_cast<OutT*>(L.out) + ((size_t)n * L.out_h + y0) * L.out_w * 3;
    const StatSlot* st = L.stats ? L.stats + (size_t)n * L.slots : nullptr;
    const int orow = L.out_w * 3;
    float gm[3], gk[3];
#pragma unroll
    for (int c = 0; c < 3; c++) {
        gm[c] = L.mean[c];
        gk[c] = L.stddev[c] > 0.f ? __fdiv_rn(L.scale, L.stddev[c]) : 0.f;
    }
    for (int e = threadIdx.x; e < rows * orow; e += 256) {
        const int r = e / orow, j = e - r * orow;
        const int y = y0 + r, x = j / 3, c = j - 3 * x;
        float v = 0.f;
        if (y < h && x < w) {
            const float px = (float)img[(size_t)y * s.src_stride + j];
            float m = c == 0 ? gm[0] : (c == 1 ? gm[1] : gm[2]);
            float k = c == 0 ? gk[0] : (c == 1 ? gk[1] : gk[2]);
            if (st) {
                const float2 mk = *reinterpret_cast<const float2*>(&st[stat_index(L.mask, y, x, c, w)]);
                m = mk.x;
                k = mk.y;
            }
            v = fmaf(sub_rn(px, m), k, L.shift);
        } else if (!L.fill_padding) {
            continue;
        }
        out[e] = OutConv<OutT>::cvt(v);
    }
}

__global__ void __launch_bounds__(256) transpose_kernel(const uint8_t* __restrict__ arena,
                                                         const rb200_pointwise_sample* __restrict__ samples, int p0, int p1,
                                                         int p2, uint8_t* __restrict__ out, int m0, int m1, int m2) {
    const int n = blockIdx.y;
    const rb200_pointwise_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset + (size_t)s.roi_y * s.src_stride + (size_t)s.roi_x * 3;
    const int d[3] = {s.roi_h, s.roi_w, 3};
    const int o0 = d[p0], o1 = d[p1], o2 = d[p2];
    const size_t total = (size_t)o0 * o1 * o2;
    uint8_t* o = out + (size_t)n * m0 * m1 * m2;
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
        const int i2 = (int)(e % o2), i1 = (int)((e / o2) % o1), i0 = (int)(e / ((size_t)o2 * o1));
        if (i0 >= m0 || i1 >= m1 || i2 >= m2) continue;
        int idx[3];
        idx[p0] = i0;
        idx[p1] = i1;
        idx[p2] = i2;
        o[((size_t)i0 * m1 + i1) * m2 + i2] = img[(size_t)idx[0] * s.src_stride + idx[1] * 3 + idx[2]];
    }
}

}  // namespace rb200

using namespace rb200;

extern "C" size_t rb200k_normalize_scratch_bytes(int n, int max_w, int max_h, int axis_mask) {
    if (n <= 0 || max_w <= 0 || max_h <= 0) return 0;
    return (size_t)n * (size_t)stat_slots(axis_mask & 7, max_w, max_h) * sizeof(StatSlot);
}

extern "C" int rb200k_normalize(const uint8_t* arena, const rb200_pointwise_sample* samples,
                                const rb200_pointwise_sample* h_samples, int n, const rb200_normalize_params* p,
                                void* scratch, size_t scratch_bytes, void* stream_v) {
    (void)h_samples;
    if (n == 0) return RB200_OK;
    if (!arena || !samples || !p || !p->out || n < 0 || p->out_w <= 0 || p->out_h <= 0) {
        set_error("rb200k_normalize: null pointer or non-positive size");
        return RB200_E_INVALID;
    }
    if (n > 65535) {
        set_error("rb200k_normalize: batch %d exceeds 65535", n);
        return RB200_E_LIMIT;
    }
    if (p->out_dtype != RB200_FP32 && p->out_dtype != RB200_FP16) {
        set_error("rb200k_normalize: the output is float32 or float16");
        return RB200_E_INVALID;
    }
    const bool computes = p->compute_mean || p->compute_stddev;
    if (computes && (p->axis_mask < 1 || p->axis_mask > 7)) {
        set_error("rb200k_normalize: axis_mask %d names no axis to reduce", p->axis_mask);
        return RB200_E_INVALID;
    }
    cudaStream_t stream = (cudaStream_t)stream_v;
    NormLaunch L;
    L.out = p->out;
    L.out_w = p->out_w;
    L.out_h = p->out_h;
    L.fp16 = p->out_dtype == RB200_FP16;
    L.mask = p->axis_mask & 7;
    L.compute_mean = p->compute_mean ? 1 : 0;
    L.compute_stddev = p->compute_stddev ? 1 : 0;
    L.fill_padding = p->fill_padding;
    for (int c = 0; c < 3; c++) { L.mean[c] = p->mean[c]; L.stddev[c] = p->stddev[c]; }
    L.scale = p->scale;
    L.shift = p->shift;
    L.stats = nullptr;
    L.slots = 0;
    L.th = 16;
    L.status = default_status_word();
    L.bounds = arena_bounds(arena, p->arena_bytes);
    if (kCheckBounds && p->arena_bytes && !L.status) {
        set_error("rb200k_normalize: the device's status word cannot be addressed");
        return RB200_E_CUDA;
    }
    if (p->out_bytes && (uint64_t)n * p->out_w * p->out_h * 3 * out_elem_size(p->out_dtype) > p->out_bytes) {
        set_error("rb200k_normalize: %d samples of %d x %d x 3 elements do not fit the %llu-byte output", n, p->out_w, p->out_h,
                  (unsigned long long)p->out_bytes);
        return RB200_E_INVALID;
    }
    const int tiles = (p->out_h + L.th - 1) / L.th;
    if (computes) {
        L.slots = stat_slots(L.mask, p->out_w, p->out_h);
        const size_t need = (size_t)n * L.slots * sizeof(StatSlot);
        if (!scratch || scratch_bytes < need) {
            set_error("rb200k_normalize: %zu bytes of scratch needed, %zu given", need, scratch ? scratch_bytes : (size_t)0);
            return RB200_E_INVALID;
        }
        L.stats = static_cast<StatSlot*>(scratch);
        int rc = check_cuda(cudaMemsetAsync(scratch, 0, need, stream), "cudaMemsetAsync(normalize scratch)");
        if (rc) return rc;
        normalize_sums_kernel<<<dim3((unsigned)tiles, (unsigned)n), 192, 0, stream>>>(arena, samples, L);
        RB200_CHECK_LAUNCH("normalize_sums_kernel");
        normalize_finish_kernel<<<(unsigned)n, 256, 0, stream>>>(samples, L);
        RB200_CHECK_LAUNCH("normalize_finish_kernel");
    }
    if (L.fp16)
        normalize_apply_kernel<__half><<<dim3((unsigned)tiles, (unsigned)n), 256, 0, stream>>>(arena, samples, L);
    else
        normalize_apply_kernel<float><<<dim3((unsigned)tiles, (unsigned)n), 256, 0, stream>>>(arena, samples, L);
    RB200_CHECK_LAUNCH("normalize_apply_kernel");
    return RB200_OK;
}

// ---- rb200k_normalize_static: the same operator with its statistics scratch inside the library image ----
//
// 65 536 slots of 16 bytes = 1 MiB of device memory, held by every GPU that loads the library until the process exits.
// In host code the array's name only stands for the device object: the address the kernels need is obtained once per
// device with cudaGetSymbolAddress while that device is current, and cached.
namespace rb200 {
constexpr size_t kStaticStatSlots = 65536;
static __device__ __align__(256) StatSlot g_static_stats[kStaticStatSlots];
static StatSlot* g_static_stats_ptr[64] = {nullptr};     // per device ordinal; written once, then only read
}  // namespace rb200

extern "C" int rb200k_normalize_static(const uint8_t* arena, const rb200_pointwise_sample* samples,
                                       const rb200_pointwise_sample* h_samples, int n, const rb200_normalize_params* p,
                                       void* stream_v) {
    if (!p) {
        set_error("rb200k_normalize_static: null parameter block");
        return RB200_E_INVALID;
    }
    const bool computes = p->compute_mean || p->compute_stddev;
    if (!computes || n <= 0) return rb200k_normalize(arena, samples, h_samples, n, p, nullptr, 0, stream_v);
    const size_t slots = (size_t)n * (size_t)stat_slots(p->axis_mask & 7, p->out_w > 0 ? p->out_w : 0, p->out_h > 0 ? p->out_h : 0);
    if (slots > kStaticStatSlots) {
        set_error("rb200k_normalize_static: this batch needs %zu statistic slots (%d samples x %zu values each for axis_mask %d "
                  "on a %d x %d output), the built-in scratch holds %zu; use rb200k_normalize with scratch of your own",
                  slots, n, slots / (size_t)n, p->axis_mask, p->out_w, p->out_h, kStaticStatSlots);
        return RB200_E_LIMIT;
    }
    int dev = -1;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev < 0 || dev >= 64) {
        set_error("rb200k_normalize_static: device ordinal %d is beyond the 64 this entry point keeps an address for", dev);
        return RB200_E_LIMIT;
    }
    StatSlot* ptr = g_static_stats_ptr[dev];
    if (!ptr) {
        // first call on this device: resolve the array's device address (the device is current)
        rc = check_cuda(cudaGetSymbolAddress((void**)&ptr, g_static_stats), "cudaGetSymbolAddress(built-in normalize scratch)");
        if (rc) return rc;
        g_static_stats_ptr[dev] = ptr;
    }
    return rb200k_normalize(arena, samples, h_samples, n, p, ptr, kStaticStatSlots * sizeof(StatSlot), stream_v);
}

extern "C" int rb200k_transpose(const uint8_t* arena, const rb200_pointwise_sample* samples, int n, const int32_t perm[3],
                                uint8_t* out, const int32_t out_dims[3], void* stream_v) {
    if (n == 0) return RB200_OK;
    if (!arena || !samples || !perm || !out || !out_dims || n < 0 || out_dims[0] <= 0 || out_dims[1] <= 0 || out_dims[2] <= 0) {
        set_error("rb200k_transpose: null pointer");
        return RB200_E_INVALID;
    }
    int seen = 0;
    for (int k = 0; k < 3; k++) {
        if (perm[k] < 0 || perm[k] > 2) { set_error("rb200k_transpose: perm[%d] = %d", k, perm[k]); return RB200_E_INVALID; }
        seen |= 1 << perm[k];
    }
    if (seen != 7) { set_error("rb200k_transpose: perm is not a permutation of 0, 1, 2"); return RB200_E_INVALID; }
    if (n > 65535) { set_error("rb200k_transpose: batch %d exceeds 65535", n); return RB200_E_LIMIT; }
    transpose_kernel<<<dim3(296, (unsigned)n), 256, 0, (cudaStream_t)stream_v>>>(arena, samples, perm[0], perm[1], perm[2], out, out_dims[0], out_dims[1],
                                                                             out_dims[2]);
    RB200_CHECK_LAUNCH("transpose_kernel");
    return RB200_OK;
}
