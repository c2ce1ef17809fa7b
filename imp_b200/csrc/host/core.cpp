#include "core.hpp"

#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <ctime>

namespace imp {

void check_launch(int rc, const char* what) {
    if (rc == 0) return;
    const std::string msg = std::string(what) + " failed (" + std::to_string(rc) + "): " + imp_last_error();
    fail(rc < 0 ? IMP_ERROR_INVALID_ARG : IMP_ERROR_CUDA, msg);
}

const char* dtype_name(int dtype) {
    switch (dtype) {
        case F32: return "float32";
        case BF16: return "bfloat16";
        case I32: return "int32";
    }
    return "?";
}

int dtype_from_name(const std::string& n) {
    if (n == "float32" || n == "fp32" || n == "f32") return F32;
    if (n == "bfloat16" || n == "bf16") return BF16;
    if (n == "int32" || n == "i32") return I32;
    fail(IMP_ERROR_INVALID_ARG, "element type must be bfloat16, float32 or int32, got '" + n + "'");
}

std::string shape_string(const Tensor& t) {
    std::string s = "[";
    for (int i = 0; i < t.ndim; ++i) s += (i ? ", " : "") + std::to_string(t.shape[i]);
    return s + "]";
}

// ------------------------------------------------------------------------------ device memory
DeviceBuffer::DeviceBuffer(size_t bytes, bool zero) : n_(bytes) {
    if (bytes == 0) return;
    cudaError_t e = cudaMalloc(&p_, bytes);
    if (e != cudaSuccess) {
        p_ = nullptr;
        n_ = 0;
        (void)cudaGetLastError();
        fail(e == cudaErrorMemoryAllocation ? IMP_ERROR_OUT_OF_MEMORY : IMP_ERROR_CUDA,
             "cannot allocate " + std::to_string(bytes) + " bytes of device memory: " + cudaGetErrorString(e));
    }
    if (zero) IMP_CUDA(cudaMemset(p_, 0, bytes));
}
DeviceBuffer::~DeviceBuffer() { reset(); }
DeviceBuffer& DeviceBuffer::operator=(DeviceBuffer&& o) noexcept {
    if (this != &o) {
        reset();
        p_ = o.p_;
        n_ = o.n_;
        o.p_ = nullptr;
        o.n_ = 0;
    }
    return *this;
}
void DeviceBuffer::reset() {
    if (p_) cudaFree(p_);
    p_ = nullptr;
    n_ = 0;
}

PinnedBuffer::PinnedBuffer(size_t bytes) : n_(bytes) {
    if (bytes == 0) return;
    cudaError_t e = cudaMallocHost(&p_, bytes);
    if (e != cudaSuccess) {
        p_ = nullptr;
        n_ = 0;
        fail(IMP_ERROR_OUT_OF_MEMORY, std::string("cannot allocate pinned host memory: ") + cudaGetErrorString(e));
    }
    memset(p_, 0, bytes);
}
PinnedBuffer::~PinnedBuffer() {
    if (p_) cudaFreeHost(p_);
}
PinnedBuffer& PinnedBuffer::operator=(PinnedBuffer&& o) noexcept {
    if (this != &o) {
        if (p_) cudaFreeHost(p_);
        p_ = o.p_;
        n_ = o.n_;
        o.p_ = nullptr;
        o.n_ = 0;
    }
    return *this;
}

// -------------------------------------------------------------------------------------- arena
static size_t align_up(size_t n, size_t a) { return (n + a - 1) / a * a; }

Arena::Arena(size_t step_bytes, size_t layer_bytes) {
    if (step_bytes) step_.main = DeviceBuffer(align_up(step_bytes, 256));
    if (layer_bytes)
        for (auto& r : layer_) r.main = DeviceBuffer(align_up(layer_bytes, 256));
}

void* Arena::Region::bump(size_t bytes, bool frozen) {
    bytes = align_up(bytes ? bytes : 1, 256);
    need += bytes;
    if (used + bytes <= main.bytes()) {
        void* p = (char*)main.data() + used;
        used += bytes;
        return p;
    }
    if (frozen)
        fail(IMP_ERROR_INTERNAL, "the workspace would have to grow while a CUDA graph is being captured");
    extra.emplace_back(bytes);
    return extra.back().data();
}

void* Arena::alloc(size_t bytes) { return layer_[cur_].bump(bytes, frozen_); }
void* Arena::alloc_step(size_t bytes) { return step_.bump(bytes, frozen_); }

void Arena::merge(Region& r, size_t& hw) {
    if (r.need > hw) hw = r.need;
    if (!r.extra.empty()) {
        // The step outgrew the block.  cudaFree waits for the device, so nothing still reads the old blocks.
        r.extra.clear();
        r.main.reset();
        r.main = DeviceBuffer(align_up(hw + hw / 8, 1 << 20));
        ++generation_;
    }
    r.used = 0;
    r.need = 0;
}

void Arena::begin_step(cudaStream_t) {
    merge(step_, hw_step_);
    // both layer regions get the size of the larger one
    size_t before = hw_layer_;
    for (auto& r : layer_) merge(r, hw_layer_);
    if (hw_layer_ > before)
        for (auto& r : layer_)
            if (r.main.bytes() < hw_layer_) {
                r.main.reset();
                r.main = DeviceBuffer(align_up(hw_layer_ + hw_layer_ / 8, 1 << 20));
                ++generation_;
            }
    cur_ = 0;
}

void Arena::next_layer() {
    cur_ ^= 1;
    merge(layer_[cur_], hw_layer_);
}

Arena::Mark Arena::mark() const {
    Mark m;
    m.step_used = step_.used;
    m.layer_used[0] = layer_[0].used;
    m.layer_used[1] = layer_[1].used;
    m.cur = cur_;
    return m;
}

void Arena::restore(const Mark& m) {
    step_.used = step_.need = m.step_used;
    for (int i = 0; i < 2; ++i) layer_[i].used = layer_[i].need = m.layer_used[i];
    cur_ = m.cur;
}

size_t Arena::capacity_bytes() const {
    size_t n = step_.main.bytes();
    for (const auto& r : layer_) n += r.main.bytes();
    return n;
}

// ------------------------------------------------------------------------------------ environment
bool env_flag(const char* name, bool dflt) {
    const char* v = getenv(name);
    if (!v || !*v) return dflt;
    return !(v[0] == '0' && v[1] == 0);
}
std::string env_string(const char* name, const std::string& dflt) {
    const char* v = getenv(name);
    return (v && *v) ? std::string(v) : dflt;
}

void log_line(LogLevel level, const char* fmt, ...) {
    static int threshold = -1;
    if (threshold < 0) {
        const std::string v = env_string("IMP_B200_LOG", "warn");
        threshold = v == "debug" ? LOG_DEBUG : v == "info" ? LOG_INFO : v == "error" ? LOG_ERROR : LOG_WARN;
    }
    if (level < threshold) return;
    static const char* names[] = {"DEBUG", "INFO", "WARN", "ERROR"};
    time_t now = time(nullptr);
    struct tm tmv;
    localtime_r(&now, &tmv);
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    fprintf(stderr, "[%02d:%02d:%02d][%s] %s\n", tmv.tm_hour, tmv.tm_min, tmv.tm_sec, names[level], buf);
}

}  // namespace imp
