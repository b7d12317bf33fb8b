/* Minimal stand-in for the OpenVX headers, enough to compile reference-owned CPU code that
 * never calls into OpenVX on the paths the oracle build uses. Test infrastructure only. */
#ifndef ORACLE_STUB_VX_H
#define ORACLE_STUB_VX_H
#include <stddef.h>
#include <stdint.h>
typedef struct _vx_reference* vx_reference;
typedef struct _vx_context* vx_context;
typedef struct _vx_graph* vx_graph;
typedef struct _vx_node* vx_node;
typedef struct _vx_tensor* vx_tensor;
typedef struct _vx_array* vx_array;
typedef struct _vx_scalar* vx_scalar;
typedef struct _vx_parameter* vx_parameter;
typedef struct _vx_image* vx_image;
typedef int32_t vx_status;
typedef int32_t vx_enum;
typedef size_t vx_size;
typedef uint8_t vx_uint8;
typedef int8_t vx_int8;
typedef int16_t vx_int16;
typedef uint16_t vx_uint16;
typedef uint32_t vx_uint32;
typedef int32_t vx_int32;
typedef uint64_t vx_uint64;
typedef int64_t vx_int64;
typedef float vx_float32;
typedef double vx_float64;
typedef uint16_t vx_float16;
typedef char vx_char;
typedef int vx_bool;
typedef uint32_t vx_df_image;
#define VX_SUCCESS 0
#define VX_CALLBACK
#define VX_API_CALL
#define VX_MAX_LOG_MESSAGE_LEN 1024
enum {
    VX_TYPE_CHAR = 1, VX_TYPE_INT8, VX_TYPE_UINT8, VX_TYPE_INT16, VX_TYPE_UINT16, VX_TYPE_INT32,
    VX_TYPE_UINT32, VX_TYPE_INT64, VX_TYPE_UINT64, VX_TYPE_FLOAT32, VX_TYPE_FLOAT64, VX_TYPE_ENUM,
    VX_TYPE_SIZE, VX_TYPE_DF_IMAGE, VX_TYPE_FLOAT16, VX_TYPE_BOOL,
    VX_MEMORY_TYPE_NONE = 100, VX_MEMORY_TYPE_HOST, VX_MEMORY_TYPE_HIP, VX_MEMORY_TYPE_OPENCL,
    VX_READ_ONLY = 200, VX_WRITE_ONLY, VX_READ_AND_WRITE,
    VX_PARAMETER_ATTRIBUTE_REF = 300, VX_PARAMETER_REF = 301
};
#ifdef __cplusplus
extern "C" {
#endif
vx_status vxReleaseNode(vx_node* node);
vx_status vxReleaseTensor(vx_tensor* t);
vx_status vxReleaseArray(vx_array* a);
vx_status vxReleaseScalar(vx_scalar* s);
vx_context vxGetContext(vx_reference ref);
vx_array vxCreateArray(vx_context ctx, vx_enum type, vx_size capacity);
vx_status vxAddArrayItems(vx_array arr, vx_size count, const void* ptr, vx_size stride);
vx_status vxCopyArrayRange(vx_array arr, vx_size start, vx_size end, vx_size stride, void* ptr, vx_enum usage, vx_enum mem);
vx_scalar vxCreateScalar(vx_context ctx, vx_enum type, const void* ptr);
vx_parameter vxGetParameterByIndex(vx_node node, vx_uint32 index);
vx_status vxQueryParameter(vx_parameter p, vx_enum attr, void* ptr, vx_size size);
vx_status vxGetStatus(vx_reference ref);
vx_status vxReadScalarValue(vx_scalar s, void* ptr);
vx_status vxWriteScalarValue(vx_scalar s, const void* ptr);
#ifdef __cplusplus
}
#endif
#endif
