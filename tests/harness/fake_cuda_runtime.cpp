// A stand-in for the CUDA runtime and for the kernel entry points, so that the host side of the library (graph
// planning, the loader thread, the ring of output slots, feeding, metadata) can be compiled with g++ and run on a
// machine without a GPU under -fsanitize=address,undefined and -fsanitize=thread. "Device" memory is ordinary heap
// memory (so the address sanitizer watches every table and buffer the host code sizes), streams execute in line, events
// are always complete. The kernels are replaced by loops that write one value per sample - the first byte of the
// sample's source window - into the sample's whole output, which is enough to see that batch k's output came from batch
// k's input through the ring.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "rb200_kernels.h"

extern "C" {

cudaError_t cudaMalloc(void** p, size_t bytes) {
    *p = std::malloc(bytes ? bytes : 1);
    return *p ? cudaSuccess : cudaErrorMemoryAllocation;
}
cudaError_t cudaFree(void* p) {
    std::free(p);
    return cudaSuccess;
}
cudaError_t cudaHostAlloc(void** p, size_t bytes, unsigned int) { return cudaMalloc(p, bytes); }
cudaError_t cudaFreeHost(void* p) { return cudaFree(p); }
cudaError_t cudaHostGetDevicePointer(void** d, void* h, unsigned int) {
    *d = h;
    return cudaSuccess;
}
cudaError_t cudaSetDevice(int) { return cudaSuccess; }
cudaError_t cudaGetDeviceCount(int* n) {
    *n = 1;
    return cudaSuccess;
}
cudaError_t cudaGetLastError(void) { return cudaSuccess; }
const char* cudaGetErrorString(cudaError_t) { return "fake CUDA runtime"; }

cudaError_t cudaStreamCreateWithFlags(cudaStream_t* s, unsigned int) {
    *s = reinterpret_cast<cudaStream_t>(std::malloc(1));
    return cudaSuccess;
}
cudaError_t cudaStreamDestroy(cudaStream_t s) {
    std::free(s);
    return cudaSuccess;
}
cudaError_t cudaStreamSynchronize(cudaStream_t) { return cudaSuccess; }
cudaError_t cudaStreamWaitEvent(cudaStream_t, cudaEvent_t, unsigned int) { return cudaSuccess; }
cudaError_t cudaEventCreateWithFlags(cudaEvent_t* e, unsigned int) {
    *e = reinterpret_cast<cudaEvent_t>(std::malloc(1));
    return cudaSuccess;
}
cudaError_t cudaEventDestroy(cudaEvent_t e) {
    std::free(e);
    return cudaSuccess;
}
cudaError_t cudaEventRecord(cudaEvent_t, cudaStream_t) { return cudaSuccess; }
cudaError_t cudaEventSynchronize(cudaEvent_t) { return cudaSuccess; }
cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t, cudaEvent_t) {
    *ms = 0.001f;
    return cudaSuccess;
}

cudaError_t cudaMemcpy(void* d, const void* s, size_t n, cudaMemcpyKind) {
    std::memcpy(d, s, n);
    return cudaSuccess;
}
cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, cudaMemcpyKind k, cudaStream_t) { return cudaMemcpy(d, s, n, k); }
cudaError_t cudaMemcpy2D(void* d, size_t dp, const void* s, size_t sp, size_t w, size_t h, cudaMemcpyKind) {
    for (size_t y = 0; y < h; y++) std::memcpy(static_cast<char*>(d) + y * dp, static_cast<const char*>(s) + y * sp, w);
    return cudaSuccess;
}
cudaError_t cudaMemcpy2DAsync(void* d, size_t dp, const void* s, size_t sp, size_t w, size_t h, cudaMemcpyKind k, cudaStream_t) {
    return cudaMemcpy2D(d, dp, s, sp, w, h, k);
}
cudaError_t cudaMemsetAsync(void* d, int v, size_t n, cudaStream_t) {
    std::memset(d, v, n);
    return cudaSuccess;
}

// ---- kernel entry points ----------------------------------------------------------------------------------

static std::atomic<uint64_t> g_launches{0};

static void fill(void* out, int dtype, size_t first, size_t count, uint8_t v) {
    if (dtype == RB200_UINT8) std::memset(static_cast<uint8_t*>(out) + first, v, count);
    else if (dtype == RB200_FP32) for (size_t i = 0; i < count; i++) static_cast<float*>(out)[first + i] = (float)v;
    else for (size_t i = 0; i < count; i++) static_cast<uint16_t*>(out)[first + i] = v;      // not a half: a tag
}

int rb200k_resample(const uint8_t* arena, const rb200_resample_sample* s, const rb200_resample_sample* hs, int n,
                    const rb200_resample_params* p, void*) {
    g_launches++;
    const size_t per = (size_t)p->out_w * p->out_h * 3;
    for (int i = 0; i < n; i++) {
        if (hs && std::memcmp(&hs[i], &s[i], sizeof(*s)) != 0) return RB200_E_INVALID;   // the two tables must agree
        fill(p->out, p->out_dtype, per * i, per, arena[s[i].src_offset + (size_t)s[i].roi_y * s[i].src_stride + (size_t)s[i].roi_x * 3]);
    }
    return RB200_OK;
}
int rb200k_resample_probe(const uint8_t* a, const rb200_resample_sample* s, const rb200_resample_sample* hs, int n,
                          const rb200_resample_params* p, void* st, uint64_t, int) {
    return rb200k_resample(a, s, hs, n, p, st);
}
int rb200k_pointwise(const uint8_t* arena, const rb200_pointwise_sample* s, const rb200_pointwise_sample* hs, int n,
                     const rb200_pointwise_params* p, void*) {
    g_launches++;
    const size_t per = (size_t)p->out_w * p->out_h * 3;
    for (int i = 0; i < n; i++) {
        if (hs && std::memcmp(&hs[i], &s[i], sizeof(*s)) != 0) return RB200_E_INVALID;
        fill(p->out, p->out_dtype, per * i, per, arena[s[i].src_offset + (size_t)s[i].roi_y * s[i].src_stride + (size_t)s[i].roi_x * 3]);
    }
    return RB200_OK;
}
int rb200k_pointwise_probe(const uint8_t* a, const rb200_pointwise_sample* s, const rb200_pointwise_sample* hs, int n,
                           const rb200_pointwise_params* p, void* st, uint64_t, int) {
    return rb200k_pointwise(a, s, hs, n, p, st);
}
int rb200k_warp_affine(const uint8_t* arena, const rb200_warp_sample* s, int n, const rb200_warp_params* p, void*) {
    g_launches++;
    const size_t per = (size_t)p->out_w * p->out_h * 3;
    for (int i = 0; i < n; i++) fill(p->out, RB200_UINT8, per * i, per, arena[s[i].src_offset]);
    return RB200_OK;
}
size_t rb200k_normalize_scratch_bytes(int n, int, int, int) { return (size_t)n * 16; }
int rb200k_normalize(const uint8_t* arena, const rb200_pointwise_sample* s, const rb200_pointwise_sample*, int n,
                     const rb200_normalize_params* p, void*, size_t, void*) {
    g_launches++;
    const size_t per = (size_t)p->out_w * p->out_h * 3;
    for (int i = 0; i < n; i++) fill(p->out, p->out_dtype, per * i, per, arena[s[i].src_offset]);
    return RB200_OK;
}
int rb200k_transpose(const uint8_t* arena, const rb200_pointwise_sample* s, int n, const int32_t*, uint8_t* out, const int32_t d[3],
                     void*) {
    g_launches++;
    const size_t per = (size_t)d[0] * d[1] * d[2];
    for (int i = 0; i < n; i++) std::memset(out + per * i, arena[s[i].src_offset], per);
    return RB200_OK;
}
int rb200k_box_encode(const float*, const int32_t*, const int32_t* offsets, int n, int, const rb200_box_encoder_params* p,
                      float* out_boxes, int32_t* out_labels, void*) {
    g_launches++;
    for (size_t i = 0; i < (size_t)n * p->num_anchors; i++) {
        out_labels[i] = offsets[i / p->num_anchors + 1] - offsets[i / p->num_anchors];    // the sample's box count
        for (int c = 0; c < 4; c++) out_boxes[i * 4 + c] = 0.f;
    }
    return RB200_OK;
}
int rb200k_box_iou_match(const float*, const int32_t*, int n, int, const rb200_box_matcher_params* p, int32_t* out, void*) {
    g_launches++;
    for (size_t i = 0; i < (size_t)n * p->num_anchors; i++) out[i] = -1;
    return RB200_OK;
}
int rb200k_device_status(void) { return 0; }
const char* rb200k_last_error(void) { return "fake kernel error"; }
uint64_t rb200k_launch_count(void) { return g_launches.load(); }
const char* rb200k_version(void) { return "rocal_b200 host-logic stand-in"; }

}  // extern "C"
