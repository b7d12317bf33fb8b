/* Stand-in for HIP's half type: __float2half rounds to nearest even, as the device instruction does.
 * Test infrastructure only. */
#ifndef ORACLE_STUB_HIP_FP16_H
#define ORACLE_STUB_HIP_FP16_H
typedef _Float16 __half;
static inline __half __float2half(float f) { return (_Float16)f; }
#endif
