/* Stand-in for the HIP runtime headers: enough to compile the reference's own device kernels
 * (rocAL/rocAL_hip/rocal_hip_kernels.cpp) for the HOST, where they lie, so that their arithmetic
 * can be run on the CPU as a pin for the restatement. TEST INFRASTRUCTURE ONLY.
 *
 * What is modelled
 *   - the vector types the kernels use (uint2/3/4, int2/4, float2/3/4) with the element-wise operators
 *     and the scalar-broadcast conversion `(float4)x` that HIP's own headers provide; a float-vector
 *     product that feeds a sum is one fused multiply-add per element (see REF_HIP_FVEC);
 *   - thread / block indices as thread-local variables that the launch loop below sets: the kernels
 *     neither synchronise nor share memory, so running the grid's threads one after another is exact;
 *   - hipLaunchKernelGGL as that loop;
 *   - __builtin_amdgcn_cvt_pk_u8_f32 (the V_CVT_PK_U8_F32 instruction): float -> uint8 with
 *     round-to-nearest-even under the default rounding mode and saturation to [0,255], packed into
 *     the selected byte. NaN converts to 0.
 * Build with -ffp-contract=fast --param=avoid-fma-max-bits=0: contraction is the HIP compiler's default
 * for device code, so a scalar a*b+c in the kernels' source is one fused multiply-add there, as it is in
 * this host build (the parameter stops gcc's x86 tuning from skipping candidates on loop-carried sums).
 */
#ifndef ORACLE_STUB_HIP_RUNTIME_H
#define ORACLE_STUB_HIP_RUNTIME_H
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline

typedef unsigned int uint;
typedef unsigned char uchar;
typedef struct ref_hip_stream* hipStream_t;

/* Integer vectors: plain element-wise structs. */
#define REF_HIP_IVEC2(NAME, T)                                                     \
    struct NAME {                                                                  \
        T x, y;                                                                    \
        NAME() = default;                                                          \
        NAME(T v) : x(v), y(v) {}                                                  \
        NAME(T a, T b) : x(a), y(b) {}                                             \
    };
#define REF_HIP_IVEC3(NAME, T)                                                     \
    struct NAME {                                                                  \
        T x, y, z;                                                                 \
        NAME() = default;                                                          \
        NAME(T v) : x(v), y(v), z(v) {}                                            \
        NAME(T a, T b, T c) : x(a), y(b), z(c) {}                                  \
    };
#define REF_HIP_IVEC4(NAME, T)                                                     \
    struct NAME {                                                                  \
        T x, y, z, w;                                                              \
        NAME() = default;                                                          \
        NAME(T v) : x(v), y(v), z(v), w(v) {}                                      \
        NAME(T a, T b, T c, T d) : x(a), y(b), z(c), w(d) {}                       \
    };

/* Float vectors. HIP's element-wise operators are inline functions, and the HIP compiler fuses a product
 * that feeds a sum after inlining (-ffp-contract=fast is its default for device code). Which of two
 * candidate products a host compiler would fuse is a tuning decision, so the rule is spelled out here
 * instead: `a * b` yields an unevaluated product, `product + c` is one fmaf per element, and a product
 * used in any other way is rounded first. */
#define REF_HIP_FVEC(NAME, PROD, N, ...)                                           \
    struct PROD;                                                                   \
    struct NAME {                                                                  \
        float __VA_ARGS__;                                                         \
        NAME() = default;                                                          \
        NAME(float v) { for (int i = 0; i < N; i++) (&x)[i] = v; }                 \
        inline NAME(const PROD& p);                                                \
        float& at(int i) { return (&x)[i]; }                                       \
        float at(int i) const { return (&x)[i]; }                                  \
    };                                                                             \
    struct PROD { NAME a, b; };                                                    \
    inline NAME::NAME(const PROD& p) { for (int i = 0; i < N; i++) (&x)[i] = p.a.at(i) * p.b.at(i); } \
    static inline PROD operator*(NAME a, NAME b) { PROD p; p.a = a; p.b = b; return p; } \
    static inline NAME operator+(NAME a, NAME b) { NAME r; for (int i = 0; i < N; i++) r.at(i) = a.at(i) + b.at(i); return r; } \
    static inline NAME operator-(NAME a, NAME b) { NAME r; for (int i = 0; i < N; i++) r.at(i) = a.at(i) - b.at(i); return r; } \
    static inline NAME operator+(const PROD& p, NAME c) { NAME r; for (int i = 0; i < N; i++) r.at(i) = fmaf(p.a.at(i), p.b.at(i), c.at(i)); return r; } \
    static inline NAME operator+(NAME c, const PROD& p) { return p + c; }

REF_HIP_FVEC(float2, ref_hip_prod2, 2, x, y)
REF_HIP_FVEC(float3, ref_hip_prod3, 3, x, y, z)
REF_HIP_FVEC(float4, ref_hip_prod4, 4, x, y, z, w)

REF_HIP_IVEC2(uint2, unsigned)
REF_HIP_IVEC3(uint3, unsigned)
REF_HIP_IVEC4(uint4, unsigned)
REF_HIP_IVEC2(int2, int)
REF_HIP_IVEC4(int4, int)

static inline uint2 make_uint2(unsigned a, unsigned b) { return uint2(a, b); }
static inline uint3 make_uint3(unsigned a, unsigned b, unsigned c) { return uint3(a, b, c); }
static inline uint4 make_uint4(unsigned a, unsigned b, unsigned c, unsigned d) { return uint4(a, b, c, d); }
static inline float2 make_float2(float a, float b) { float2 r; r.x = a; r.y = b; return r; }
static inline float3 make_float3(float a, float b, float c) { float3 r; r.x = a; r.y = b; r.z = c; return r; }
static inline float4 make_float4(float a, float b, float c, float d) { float4 r; r.x = a; r.y = b; r.z = c; r.w = d; return r; }

struct dim3 {
    unsigned x, y, z;
    dim3(unsigned a = 1, unsigned b = 1, unsigned c = 1) : x(a), y(b), z(c) {}
};

static thread_local unsigned hipBlockIdx_x, hipBlockIdx_y, hipBlockIdx_z;
static thread_local unsigned hipThreadIdx_x, hipThreadIdx_y, hipThreadIdx_z;
static thread_local unsigned hipBlockDim_x, hipBlockDim_y, hipBlockDim_z;
static thread_local unsigned hipGridDim_x, hipGridDim_y, hipGridDim_z;

/* The whole grid, one thread after another (z slowest). */
template <class Body>
static inline void ref_hip_launch(dim3 grid, dim3 block, Body body) {
    hipGridDim_x = grid.x; hipGridDim_y = grid.y; hipGridDim_z = grid.z;
    hipBlockDim_x = block.x; hipBlockDim_y = block.y; hipBlockDim_z = block.z;
    for (unsigned bz = 0; bz < grid.z; bz++)
        for (unsigned by = 0; by < grid.y; by++)
            for (unsigned bx = 0; bx < grid.x; bx++)
                for (unsigned tz = 0; tz < block.z; tz++)
                    for (unsigned ty = 0; ty < block.y; ty++)
                        for (unsigned tx = 0; tx < block.x; tx++) {
                            hipBlockIdx_x = bx; hipBlockIdx_y = by; hipBlockIdx_z = bz;
                            hipThreadIdx_x = tx; hipThreadIdx_y = ty; hipThreadIdx_z = tz;
                            body();
                        }
}
#define hipLaunchKernelGGL(kernel, grid, block, shared_bytes, stream, ...) \
    ref_hip_launch((grid), (block), [&]() { kernel(__VA_ARGS__); })

static inline unsigned ref_hip_cvt_pk_u8_f32(float v, unsigned byte, unsigned old) {
    float r = nearbyintf(v);           /* round to nearest even (default rounding mode) */
    unsigned q = !(r > 0.f) ? 0u : (r > 255.f ? 255u : (unsigned)r);
    const unsigned shift = 8u * (byte & 3u);
    return (old & ~(0xffu << shift)) | (q << shift);
}
#define __builtin_amdgcn_cvt_pk_u8_f32 ref_hip_cvt_pk_u8_f32

#endif
