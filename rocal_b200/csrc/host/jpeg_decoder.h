// JPEG front-end of the external source: batched decode straight into the packed device arena that the
// augmentation kernels read (the place of the reference's decoders, rocAL/source/decoders/image/
// turbo_jpeg_decoder.cpp and rocjpeg_decoder.cpp, fed by loaders/image/image_read_and_decode.cpp:287-400).
//
// The decode itself is NVIDIA's nvJPEG library, loaded with dlopen when the first compressed batch arrives
// (the library is optional: without it the raw-pixel path keeps working and a compressed feed reports an
// error). Output format is interleaved RGB, one image after the other, row pitch = width * 3.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace rb200 {

class JpegDecoder {
   public:
    JpegDecoder() = default;
    ~JpegDecoder();
    JpegDecoder(const JpegDecoder&) = delete;
    JpegDecoder& operator=(const JpegDecoder&) = delete;

    // Loads nvJPEG and creates the codec state; throws std::runtime_error with the reason on failure.
    void init();
    bool ready() const { return _handle != nullptr; }
    const char* backend_name() const { return _backend_name; }

    // Width and height of one encoded image (header parse on the host).
    void image_size(const unsigned char* data, size_t length, int& width, int& height);

    // Decodes n images to interleaved RGB. dst[i] is a device pointer with room for height*pitch[i] bytes.
    void decode_batch(const unsigned char* const* data, const size_t* lengths, int n, unsigned char* const* dst,
                      const size_t* pitch, cudaStream_t stream);

   private:
    void* _lib = nullptr;
    void* _handle = nullptr;
    void* _state = nullptr;
    int _batch_initialised = 0;
    const char* _backend_name = "none";
    // entry points resolved from the library
    void* _fn[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
};

}  // namespace rb200
