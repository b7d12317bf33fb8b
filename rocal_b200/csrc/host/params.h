// Per-batch augmentation parameters: deterministic values and seeded random generators.
//
// Behaviour follows the reference's parameter machinery so that a pipeline built with the same
// seed draws the same per-sample tables:
//   * UniformRand / CustomRand: std::mt19937(seed); one draw in the constructor; a renewal fills a
//     batch-sized array when one was requested, else one value; value = raw/max*(end-start)+start
//     in double (rocAL/include/parameters/parameter_random.h:37-239).
//   * ParameterFactory: process-wide; set_seed(s) builds a 1024-entry table from std::seed_seq{s}
//     and parameters created through the API take successive entries
//     (rocAL/source/parameters/parameter_factory.cpp:107-133); generators created as node defaults
//     are seeded with the raw seed (rocAL/include/parameters/parameter_factory.h:79-84).
#pragma once

#include <algorithm>
#include <cstdint>
#include <mutex>
#include <numeric>
#include <random>
#include <set>
#include <vector>

namespace rb200 {

template <typename T>
class Parameter {
   public:
    virtual ~Parameter() = default;
    virtual T get() = 0;
    virtual const std::vector<T>& array() = 0;
    virtual void renew() = 0;
    virtual void create_array(unsigned n) = 0;
    virtual bool single_value() const = 0;
};

template <typename T>
class SimpleParameter : public Parameter<T> {
   public:
    explicit SimpleParameter(T v) : _val(v) {}
    T get() override { return _val; }
    const std::vector<T>& array() override { return _values; }
    void renew() override {}
    void create_array(unsigned n) override {
        if (_values.empty()) _values.resize(n);
        std::fill(_values.begin(), _values.end(), _val);
    }
    bool single_value() const override { return true; }
    void update(T v) {
        _val = v;
        std::fill(_values.begin(), _values.end(), _val);
    }

   private:
    T _val;
    std::vector<T> _values;
};

template <typename T>
class UniformRand : public Parameter<T> {
   public:
    UniformRand(T start, T end, unsigned seed) : _gen(seed) {
        update(start, end);
        renew();
    }
    T get() override { return _val; }
    const std::vector<T>& array() override { return _values; }
    void renew() override {
        if (_values.empty()) {
            draw();
        } else {
            for (auto& v : _values) {
                draw();
                v = _val;
            }
        }
    }
    void create_array(unsigned n) override {
        if (_values.empty()) _values.resize(n);
    }
    bool single_value() const override { return _start == _end; }
    void update(T start, T end) {
        std::lock_guard<std::mutex> lk(_lock);
        if (end < start) end = start;
        _start = start;
        _end = end;
    }

   private:
    void draw() {
        std::lock_guard<std::mutex> lk(_lock);
        auto raw = _gen();
        if (_start == _end)
            _val = _start;
        else
            _val = static_cast<T>(((double)raw / (double)_gen.max()) * ((double)_end - (double)_start) + (double)_start);
    }
    T _start{}, _end{}, _val{};
    std::vector<T> _values;
    std::mt19937 _gen;
    std::mutex _lock;
};

template <typename T>
class CustomRand : public Parameter<T> {
   public:
    CustomRand(const T* values, const double* freqs, size_t size, unsigned seed) : _gen(seed) {
        update(values, freqs, size);
        renew();
    }
    int update(const T* values, const double* freqs, size_t size) {
        std::lock_guard<std::mutex> lk(_lock);
        if (size == 0) return -1;
        _vals.assign(values, values + size);
        std::vector<double> f(freqs, freqs + size);
        double sum = 0;
        for (auto& x : f) {
            if (x < 0) x = 0;
            sum += x;
        }
        _cdf.resize(size);
        double acc = 0;
        for (size_t i = 0; i < size; i++) {
            acc += f[i] / sum;
            _cdf[i] = acc;
        }
        return 0;
    }
    T get() override { return _val; }
    const std::vector<T>& array() override { return _values; }
    void renew() override {
        if (_values.empty()) {
            draw();
        } else {
            for (auto& v : _values) {
                draw();
                v = _val;
            }
        }
    }
    void create_array(unsigned n) override {
        if (_values.empty()) _values.resize(n);
    }
    bool single_value() const override { return _vals.size() == 1; }

   private:
    void draw() {
        std::lock_guard<std::mutex> lk(_lock);
        if (_vals.size() == 1) {
            _val = _vals[0];
            return;
        }
        double r = (double)_gen() / (double)_gen.max();
        size_t idx = std::upper_bound(_cdf.begin(), _cdf.end(), r) - _cdf.begin();
        if (idx >= _vals.size()) idx = _vals.size() - 1;
        _val = _vals[idx];
    }
    std::vector<T> _vals;
    std::vector<double> _cdf;
    T _val{};
    std::vector<T> _values;
    std::mt19937 _gen;
    std::mutex _lock;
};

enum class ParamKind { DETERMINISTIC = 0, RANDOM_UNIFORM = 1, RANDOM_CUSTOM = 2 };

// What a RocalIntParam / RocalFloatParam handle points to.
template <typename T>
struct ParamHandle {
    Parameter<T>* core;
    ParamKind kind;
};
using IntParam = ParamHandle<int>;
using FloatParam = ParamHandle<float>;

class ParameterFactory {
   public:
    static constexpr int kMaxSeeds = 1024;
    static ParameterFactory& instance();

    void set_seed(unsigned seed);
    unsigned get_seed() const { return (unsigned)_seed; }
    void renew_parameters();

    IntParam* create_uniform_int(int start, int end);
    FloatParam* create_uniform_float(float start, float end);
    IntParam* create_custom_int(const int* values, const double* freqs, size_t n);
    FloatParam* create_custom_float(const float* values, const double* freqs, size_t n);
    IntParam* create_int(int v);
    FloatParam* create_float(float v);

    // Node defaults: seeded with the raw seed, not with the seed table.
    Parameter<int>* default_uniform_int(int start, int end);
    Parameter<float>* default_uniform_float(float start, float end);
    Parameter<int>* default_int(int v);
    Parameter<float>* default_float(float v);

    bool owns(const void* handle);
    // Per-sample values of every parameter that currently holds an array of n values (what a batch was built with).
    void snapshot(size_t n, std::vector<std::pair<const void*, std::vector<int>>>& ints,
                  std::vector<std::pair<const void*, std::vector<float>>>& floats);

    ~ParameterFactory();

   private:
    ParameterFactory();
    int64_t next_seed();
    std::mutex _mutex;
    unsigned long long _seed = 0;
    std::vector<int64_t> _seed_table;
    int _seed_idx = 0;
    std::vector<Parameter<int>*> _ints;
    std::vector<Parameter<float>*> _floats;
    std::set<const void*> _handles;
};

}  // namespace rb200
