#include "params.h"

namespace rb200 {

ParameterFactory& ParameterFactory::instance() {
    static ParameterFactory f;
    return f;
}

ParameterFactory::ParameterFactory() {
    std::random_device rd;
    set_seed(rd());
}

// Parameters and their handles live as long as the process: a handle may be created before any context exists and be
// shared by several.
ParameterFactory::~ParameterFactory() {
    for (auto* p : _ints) delete p;
    for (auto* p : _floats) delete p;
    for (const void* h : _handles) ::operator delete(const_cast<void*>(h));
}

void ParameterFactory::set_seed(unsigned seed) {
    std::lock_guard<std::mutex> lk(_mutex);
    _seed = seed;
    _seed_table.assign(kMaxSeeds, 0);
    std::seed_seq ss{seed};
    ss.generate(_seed_table.begin(), _seed_table.end());
}

int64_t ParameterFactory::next_seed() {
    int64_t s = _seed_table[_seed_idx];
    _seed_idx = (_seed_idx + 1) % kMaxSeeds;
    return s;
}

void ParameterFactory::renew_parameters() {
    std::lock_guard<std::mutex> lk(_mutex);
    for (auto* p : _ints) p->renew();
    for (auto* p : _floats) p->renew();
}

IntParam* ParameterFactory::create_uniform_int(int start, int end) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new UniformRand<int>(start, end, (unsigned)next_seed());
    _ints.push_back(g);
    auto* h = new IntParam{g, ParamKind::RANDOM_UNIFORM};
    _handles.insert(h);
    return h;
}

FloatParam* ParameterFactory::create_uniform_float(float start, float end) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new UniformRand<float>(start, end, (unsigned)next_seed());
    _floats.push_back(g);
    auto* h = new FloatParam{g, ParamKind::RANDOM_UNIFORM};
    _handles.insert(h);
    return h;
}

IntParam* ParameterFactory::create_custom_int(const int* values, const double* freqs, size_t n) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new CustomRand<int>(values, freqs, n, (unsigned)next_seed());
    _ints.push_back(g);
    auto* h = new IntParam{g, ParamKind::RANDOM_CUSTOM};
    _handles.insert(h);
    return h;
}

FloatParam* ParameterFactory::create_custom_float(const float* values, const double* freqs, size_t n) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new CustomRand<float>(values, freqs, n, (unsigned)next_seed());
    _floats.push_back(g);
    auto* h = new FloatParam{g, ParamKind::RANDOM_CUSTOM};
    _handles.insert(h);
    return h;
}

IntParam* ParameterFactory::create_int(int v) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new SimpleParameter<int>(v);
    _ints.push_back(g);
    auto* h = new IntParam{g, ParamKind::DETERMINISTIC};
    _handles.insert(h);
    return h;
}

FloatParam* ParameterFactory::create_float(float v) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new SimpleParameter<float>(v);
    _floats.push_back(g);
    auto* h = new FloatParam{g, ParamKind::DETERMINISTIC};
    _handles.insert(h);
    return h;
}

Parameter<int>* ParameterFactory::default_uniform_int(int start, int end) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new UniformRand<int>(start, end, (unsigned)_seed);
    _ints.push_back(g);
    return g;
}

Parameter<float>* ParameterFactory::default_uniform_float(float start, float end) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new UniformRand<float>(start, end, (unsigned)_seed);
    _floats.push_back(g);
    return g;
}

Parameter<int>* ParameterFactory::default_int(int v) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new SimpleParameter<int>(v);
    _ints.push_back(g);
    return g;
}

Parameter<float>* ParameterFactory::default_float(float v) {
    std::lock_guard<std::mutex> lk(_mutex);
    auto* g = new SimpleParameter<float>(v);
    _floats.push_back(g);
    return g;
}

void ParameterFactory::snapshot(size_t n, std::vector<std::pair<const void*, std::vector<int>>>& ints,
                                std::vector<std::pair<const void*, std::vector<float>>>& floats) {
    std::lock_guard<std::mutex> lk(_mutex);
    ints.clear();
    floats.clear();
    for (auto* p : _ints)
        if (p->array().size() == n) ints.emplace_back(p, p->array());
    for (auto* p : _floats)
        if (p->array().size() == n) floats.emplace_back(p, p->array());
}

bool ParameterFactory::owns(const void* handle) {
    std::lock_guard<std::mutex> lk(_mutex);
    return _handles.count(handle) != 0;
}

}  // namespace rb200
