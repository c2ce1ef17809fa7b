// Core types of the host: errors, tensor views, device memory, the workspace, the runtime a part
// is built with.  The reference's counterparts are src/core/tensor.h:28-65 (a descriptor over raw
// memory) and the persistent workspaces of src/graph/executor_workspace.cu:347-408, 2048-2100.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "imp_b200/imp.h"
#include "imp_b200/imp_parts.h"
#include "json.hpp"

namespace imp {

// An error with the C API's code; every entry point turns it into (code, message).
struct Error : std::runtime_error {
    ImpError code;
    Error(ImpError c, const std::string& msg) : std::runtime_error(msg), code(c) {}
};
[[noreturn]] inline void fail(ImpError c, const std::string& msg) { throw Error(c, msg); }

#define IMP_CUDA(expr)                                                                                  \
    do {                                                                                                \
        cudaError_t e__ = (expr);                                                                       \
        if (e__ != cudaSuccess)                                                                         \
            throw ::imp::Error(e__ == cudaErrorMemoryAllocation ? IMP_ERROR_OUT_OF_MEMORY : IMP_ERROR_CUDA, \
                               std::string(#expr) + ": " + cudaGetErrorString(e__));                    \
    } while (0)

// Launchers of this library return 0, a negative argument error, or a cudaError_t; the text is in
// imp_last_error().  -2 means "this kernel does not take the shape" and is the caller's to handle.
void check_launch(int rc, const char* what);
extern "C" const char* imp_last_error(void);

// ------------------------------------------------------------------------------------ tensors
using Tensor = ImpTensor;

enum : int { F32 = IMP_ELEM_F32, BF16 = IMP_ELEM_BF16, I32 = IMP_ELEM_I32 };

inline size_t elem_size(int dtype) { return dtype == BF16 ? 2 : 4; }
const char* dtype_name(int dtype);
int dtype_from_name(const std::string& name);   // "float32"/"fp32", "bfloat16"/"bf16", "int32"; throws

inline Tensor tensor2d(void* data, int dtype, int64_t rows, int64_t cols, int64_t stride = -1) {
    Tensor t{};
    t.data = data;
    t.dtype = dtype;
    t.ndim = 2;
    t.shape[0] = rows;
    t.shape[1] = cols;
    t.stride0 = stride < 0 ? cols : stride;
    return t;
}
inline Tensor tensor_nd(void* data, int dtype, const std::vector<int64_t>& shape) {
    Tensor t{};
    t.data = data;
    t.dtype = dtype;
    t.ndim = (int)shape.size();
    int64_t inner = 1;
    for (int i = 0; i < t.ndim; ++i) {
        t.shape[i] = shape[(size_t)i];
        if (i > 0) inner *= shape[(size_t)i];
    }
    t.stride0 = inner;
    return t;
}
inline int64_t numel(const Tensor& t) {
    int64_t n = 1;
    for (int i = 0; i < t.ndim; ++i) n *= t.shape[i];
    return n;
}
inline int64_t rows(const Tensor& t) { return t.ndim ? t.shape[0] : 1; }
inline int64_t cols(const Tensor& t) { return t.ndim ? numel(t) / (t.shape[0] ? t.shape[0] : 1) : 1; }
inline bool contiguous(const Tensor& t) { return t.stride0 == cols(t); }
// Columns [c0, c0 + n) of a 2-D tensor.
inline Tensor col_slice(const Tensor& t, int64_t c0, int64_t n) {
    Tensor s = t;
    s.data = (char*)t.data + c0 * (int64_t)elem_size(t.dtype);
    s.ndim = 2;
    s.shape[0] = rows(t);
    s.shape[1] = n;
    return s;
}
// Rows [0, n) of a tensor.
inline Tensor first_rows(const Tensor& t, int64_t n) {
    Tensor s = t;
    s.shape[0] = n;
    return s;
}
std::string shape_string(const Tensor& t);

// ------------------------------------------------------------------------------ device memory
// One cudaMalloc'ed block, freed with the object.
class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes, bool zero = false);
    ~DeviceBuffer();
    DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    void* data() const { return p_; }
    size_t bytes() const { return n_; }
    void reset();

private:
    void* p_ = nullptr;
    size_t n_ = 0;
};

// Page-locked host memory.
class PinnedBuffer {
public:
    PinnedBuffer() = default;
    explicit PinnedBuffer(size_t bytes);
    ~PinnedBuffer();
    PinnedBuffer(PinnedBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
    PinnedBuffer& operator=(PinnedBuffer&& o) noexcept;
    PinnedBuffer(const PinnedBuffer&) = delete;
    void* data() const { return p_; }
    size_t bytes() const { return n_; }

private:
    void* p_ = nullptr;
    size_t n_ = 0;
};

// The workspace of the step function: every activation of a step comes from here, nothing is
// allocated per operation.  Three regions with bump allocation: `step` lives for the whole step
// (the residual stream, the logits), and two `layer` regions that alternate from layer to layer,
// so that what a layer leaves pending for the next one survives exactly one layer.  All work of a
// step is ordered on one stream, so memory is reused as soon as the host has moved on.
//
// The arena starts from an estimate by the token budget and grows when a step needs more (a new
// block, outside graph capture only); at the next step boundary the blocks are merged into one.
// `generation` changes whenever addresses may have changed: captured graphs are dropped then.
class Arena {
public:
    explicit Arena(size_t step_bytes = 0, size_t layer_bytes = 0);
    void* alloc(size_t bytes);                 // from the current layer region
    void* alloc_step(size_t bytes);            // from the step region
    void begin_step(cudaStream_t stream);      // reset everything; merge blocks if the last step grew
    void next_layer();                         // switch to the other layer region and empty it
    void freeze(bool on) { frozen_ = on; }     // while a graph is captured: growing is an error
    // Where the allocation cursors stand.  A replayed graph does not allocate on the host, so whoever replays
    // one puts the cursors where they stood when its capture ended: what is allocated after the replay must
    // not land on memory the graph's kernels use.
    struct Mark {
        size_t step_used = 0, layer_used[2] = {0, 0};
        int cur = 0;
    };
    Mark mark() const;
    void restore(const Mark& m);
    uint64_t generation() const { return generation_; }
    size_t capacity_bytes() const;
    size_t high_water_bytes() const { return hw_step_ + 2 * hw_layer_; }

    template <typename T = void> T* take(size_t count, bool step = false) {
        return (T*)(step ? alloc_step(count * sizeof(T)) : alloc(count * sizeof(T)));
    }

private:
    struct Region {
        DeviceBuffer main;
        std::vector<DeviceBuffer> extra;   // blocks added during a step
        size_t used = 0, extra_used = 0, need = 0;
        void* bump(size_t bytes, bool frozen);
        void reset() { used = 0; }
    };
    void merge(Region& r, size_t& hw);
    Region step_, layer_[2];
    int cur_ = 0;
    bool frozen_ = false;
    uint64_t generation_ = 1;
    size_t hw_step_ = 0, hw_layer_ = 0;
};

// What every part is built with and runs against.
struct Runtime {
    int dtype = BF16;               // activations and cache: BF16 or F32
    int device = 0;
    cudaStream_t stream = nullptr;
    int32_t* status = nullptr;      // device status word
    Arena* arena = nullptr;
    int sm_count = 0;
    int64_t fallback_calls = 0;     // matrix products that ran on the plain fallback kernel
    int64_t launches = 0;           // launcher calls of this library
    int64_t split_norm_calls = 0;   // norms that added the unsummed parts of a product themselves
    // IMP_B200_TIME_WITHOUT: letters of built-in operations that are NOT launched (q: q,k,v product, a: decode
    // attention, o: output product, g: gate/up product, d: down product, n: the blocks' norms).  The results are then
    // meaningless; the step's time against the full step's is what the operation costs inside the step.  A
    // measurement aid only: the context warns when it is set.
    std::string time_without;
    bool without(char op) const { return !time_without.empty() && time_without.find(op) != std::string::npos; }
    bool is_f32() const { return dtype == F32; }
    Tensor empty(int64_t rows, int64_t cols, int dt = -1, bool step = false) {
        const int d = dt < 0 ? dtype : dt;
        void* p = step ? arena->alloc_step((size_t)(rows * cols) * elem_size(d))
                       : arena->alloc((size_t)(rows * cols) * elem_size(d));
        return tensor2d(p, d, rows, cols);
    }
};

// Environment switches, read once.
bool env_flag(const char* name, bool dflt);
std::string env_string(const char* name, const std::string& dflt);

// Logging in the reference's shape: [HH:MM:SS][LEVEL] text (src/core/logging.cpp:27-56); WARN and
// above go to stderr always, INFO and DEBUG when IMP_B200_LOG names them.
enum LogLevel { LOG_DEBUG = 0, LOG_INFO = 1, LOG_WARN = 2, LOG_ERROR = 3 };
void log_line(LogLevel level, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

}  // namespace imp
