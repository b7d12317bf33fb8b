#include "jpeg_decoder.h"

#include <dlfcn.h>
#include <nvjpeg.h>

#include <cstdlib>
#include <cstring>
#include <stdexcept>

namespace rb200 {

namespace {

enum Fn { CREATE_EX = 0, DESTROY, STATE_CREATE, STATE_DESTROY, GET_INFO, BATCH_INIT, BATCH_DECODE, CREATE_SIMPLE };

using create_ex_t = nvjpegStatus_t (*)(nvjpegBackend_t, nvjpegDevAllocator_t*, nvjpegPinnedAllocator_t*, unsigned int, nvjpegHandle_t*);
using create_simple_t = nvjpegStatus_t (*)(nvjpegHandle_t*);
using destroy_t = nvjpegStatus_t (*)(nvjpegHandle_t);
using state_create_t = nvjpegStatus_t (*)(nvjpegHandle_t, nvjpegJpegState_t*);
using state_destroy_t = nvjpegStatus_t (*)(nvjpegJpegState_t);
using get_info_t = nvjpegStatus_t (*)(nvjpegHandle_t, const unsigned char*, size_t, int*, nvjpegChromaSubsampling_t*, int*, int*);
using batch_init_t = nvjpegStatus_t (*)(nvjpegHandle_t, nvjpegJpegState_t, int, int, nvjpegOutputFormat_t);
using batch_decode_t = nvjpegStatus_t (*)(nvjpegHandle_t, nvjpegJpegState_t, const unsigned char* const*, const size_t*, nvjpegImage_t*,
                                          cudaStream_t);

void fail(const std::string& what, int status) {
    throw std::runtime_error("nvJPEG: " + what + " failed with status " + std::to_string(status));
}

}  // namespace

JpegDecoder::~JpegDecoder() {
    if (_state) reinterpret_cast<state_destroy_t>(_fn[STATE_DESTROY])(static_cast<nvjpegJpegState_t>(_state));
    if (_handle) reinterpret_cast<destroy_t>(_fn[DESTROY])(static_cast<nvjpegHandle_t>(_handle));
    // the library stays loaded: other contexts of the process may use it
}

void JpegDecoder::init() {
    if (_handle) return;
    const char* names[] = {"libnvjpeg.so.12", "libnvjpeg.so"};
    for (const char* nm : names) {
        _lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
        if (_lib) break;
    }
    if (!_lib) throw std::runtime_error("compressed input needs NVIDIA's nvJPEG library (libnvjpeg.so.12), which could not be loaded");
    const char* syms[] = {"nvjpegCreateEx", "nvjpegDestroy", "nvjpegJpegStateCreate", "nvjpegJpegStateDestroy", "nvjpegGetImageInfo",
                          "nvjpegDecodeBatchedInitialize", "nvjpegDecodeBatched", "nvjpegCreateSimple"};
    for (int i = 0; i < 8; i++) {
        _fn[i] = dlsym(_lib, syms[i]);
        if (!_fn[i]) throw std::runtime_error(std::string("nvJPEG: symbol not found: ") + syms[i]);
    }
    // GPU-assisted Huffman decode for batches by default; RB200_NVJPEG_BACKEND=hardware asks for the fixed-function
    // engine, =hybrid for Huffman decode on the host. Every choice falls back to the library's default.
    nvjpegBackend_t want = NVJPEG_BACKEND_GPU_HYBRID;
    _backend_name = "gpu_hybrid";
    if (const char* e = getenv("RB200_NVJPEG_BACKEND")) {
        if (!strcmp(e, "hardware")) { want = NVJPEG_BACKEND_HARDWARE; _backend_name = "hardware"; }
        else if (!strcmp(e, "hybrid")) { want = NVJPEG_BACKEND_HYBRID; _backend_name = "hybrid"; }
        else if (!strcmp(e, "default")) { want = NVJPEG_BACKEND_DEFAULT; _backend_name = "default"; }
    }
    nvjpegHandle_t h = nullptr;
    nvjpegStatus_t st = reinterpret_cast<create_ex_t>(_fn[CREATE_EX])(want, nullptr, nullptr, NVJPEG_FLAGS_DEFAULT, &h);
    if (st != NVJPEG_STATUS_SUCCESS) {
        _backend_name = "default";
        st = reinterpret_cast<create_simple_t>(_fn[CREATE_SIMPLE])(&h);
        if (st != NVJPEG_STATUS_SUCCESS) fail("nvjpegCreateSimple", (int)st);
    }
    nvjpegJpegState_t s = nullptr;
    st = reinterpret_cast<state_create_t>(_fn[STATE_CREATE])(h, &s);
    if (st != NVJPEG_STATUS_SUCCESS) {
        reinterpret_cast<destroy_t>(_fn[DESTROY])(h);
        fail("nvjpegJpegStateCreate", (int)st);
    }
    _handle = h;
    _state = s;
}

void JpegDecoder::image_size(const unsigned char* data, size_t length, int& width, int& height) {
    int comps = 0;
    nvjpegChromaSubsampling_t sub;
    int w[NVJPEG_MAX_COMPONENT] = {0}, h[NVJPEG_MAX_COMPONENT] = {0};
    nvjpegStatus_t st = reinterpret_cast<get_info_t>(_fn[GET_INFO])(static_cast<nvjpegHandle_t>(_handle), data, length, &comps, &sub, w, h);
    if (st != NVJPEG_STATUS_SUCCESS) fail("nvjpegGetImageInfo (not a JPEG stream?)", (int)st);
    width = w[0];
    height = h[0];
}

void JpegDecoder::decode_batch(const unsigned char* const* data, const size_t* lengths, int n, unsigned char* const* dst,
                               const size_t* pitch, cudaStream_t stream) {
    nvjpegHandle_t h = static_cast<nvjpegHandle_t>(_handle);
    nvjpegJpegState_t s = static_cast<nvjpegJpegState_t>(_state);
    if (_batch_initialised != n) {
        nvjpegStatus_t st = reinterpret_cast<batch_init_t>(_fn[BATCH_INIT])(h, s, n, 1, NVJPEG_OUTPUT_RGBI);
        if (st != NVJPEG_STATUS_SUCCESS) fail("nvjpegDecodeBatchedInitialize", (int)st);
        _batch_initialised = n;
    }
    std::vector<nvjpegImage_t> out((size_t)n);
    for (int i = 0; i < n; i++) {
        std::memset(&out[i], 0, sizeof(nvjpegImage_t));
        out[i].channel[0] = dst[i];
        out[i].pitch[0] = pitch[i];
    }
    nvjpegStatus_t st = reinterpret_cast<batch_decode_t>(_fn[BATCH_DECODE])(h, s, data, lengths, out.data(), stream);
    if (st != NVJPEG_STATUS_SUCCESS) fail("nvjpegDecodeBatched", (int)st);
}

}  // namespace rb200
