/* Stand-in for half/half.hpp: the reference headers only name half_float::half. */
#ifndef ORACLE_STUB_HALF_HPP
#define ORACLE_STUB_HALF_HPP
namespace half_float {
struct half {
    _Float16 v;
    half() : v(0) {}
    half(float f) : v((_Float16)f) {}
    operator float() const { return (float)v; }
};
}  // namespace half_float
#endif
