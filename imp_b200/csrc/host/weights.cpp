#include "weights.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <set>
#include <sstream>
#include <thread>

#include "kernels.h"

namespace imp {

namespace {
[[noreturn]] void bad_file(const std::string& msg) { fail(IMP_ERROR_INVALID_MODEL, msg); }

int stored_size(const std::string& dt) {
    if (dt == "F32" || dt == "I32") return 4;
    if (dt == "BF16" || dt == "F16" || dt == "I16") return 2;
    if (dt == "F64" || dt == "I64") return 8;
    if (dt == "I8" || dt == "U8" || dt == "BOOL") return 1;
    return 0;
}
bool file_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}
std::string shape_str(const std::vector<int64_t>& s) {
    std::string o = "[";
    for (size_t i = 0; i < s.size(); ++i) o += (i ? ", " : "") + std::to_string(s[i]);
    return o + "]";
}
}  // namespace

// ---------------------------------------------------------------------------------- container
SafetensorsFile::SafetensorsFile(const std::string& path) : path_(path) {
    int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) fail(IMP_ERROR_FILE_NOT_FOUND, path + ": cannot open");
    struct stat st;
    fstat(fd, &st);
    size_ = (size_t)st.st_size;
    if (size_ < 8) {
        close(fd);
        bad_file(path + ": truncated (only " + std::to_string(size_) + " bytes)");
    }
    map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map_ == MAP_FAILED) {
        map_ = nullptr;
        fail(IMP_ERROR_INTERNAL, path + ": cannot map the file");
    }
    const uint8_t* base = (const uint8_t*)map_;
    uint64_t hlen = 0;
    memcpy(&hlen, base, 8);
    if (hlen == 0 || 8 + hlen > size_)
        bad_file(path + ": header length " + std::to_string(hlen) + " exceeds the file size " + std::to_string(size_) +
                 " (truncated file?)");
    Json header;
    try {
        header = Json::parse(std::string((const char*)base + 8, (size_t)hlen), path + ": header");
    } catch (const std::exception& e) {
        bad_file(e.what());
    }
    if (!header.is_object()) bad_file(path + ": header must be a JSON object");
    const size_t data_start = 8 + (size_t)hlen, data_size = size_ - data_start;
    for (const auto& m : header.members()) {
        if (m.first == "__metadata__") {
            if (m.second.is_object()) metadata_ = m.second;
            continue;
        }
        StoredTensor t;
        int64_t b = 0, e = 0;
        try {
            t.dtype = m.second.at("dtype").as_string();
            for (const auto& d : m.second.at("shape").items()) t.shape.push_back(d.as_int());
            const auto& off = m.second.at("data_offsets").items();
            if (off.size() != 2) throw std::runtime_error("offsets");
            b = off[0].as_int();
            e = off[1].as_int();
        } catch (const std::exception&) {
            bad_file(path + ": malformed entry for tensor '" + m.first + "'");
        }
        const int isz = stored_size(t.dtype);
        if (!isz) bad_file(path + ": tensor '" + m.first + "' has unsupported dtype " + t.dtype);
        if (b < 0 || e < b || (size_t)e > data_size)
            bad_file(path + ": tensor '" + m.first + "' data range [" + std::to_string(b) + "," + std::to_string(e) +
                     ") lies outside the file's data section of " + std::to_string(data_size) + " bytes (truncated file?)");
        int64_t n = 1;
        for (int64_t d : t.shape) n *= d;
        if (e - b != n * isz)
            bad_file(path + ": tensor '" + m.first + "' has " + std::to_string(e - b) + " bytes but shape " +
                     shape_str(t.shape) + " of " + t.dtype + " needs " + std::to_string(n * isz));
        t.data = base + data_start + b;
        t.bytes = (size_t)(e - b);
        tensors_.emplace_back(m.first, t);
    }
}

SafetensorsFile::~SafetensorsFile() {
    if (map_) munmap(map_, size_);
}

std::vector<std::unique_ptr<SafetensorsFile>> open_model_files(const std::string& folder) {
    const std::string single = folder + "/model.safetensors", index = folder + "/model.safetensors.index.json";
    std::vector<std::unique_ptr<SafetensorsFile>> out;
    if (file_exists(index)) {
        std::ifstream f(index, std::ios::binary);
        std::stringstream ss;
        ss << f.rdbuf();
        Json j;
        try {
            j = Json::parse(ss.str(), index);
        } catch (const std::exception& e) {
            bad_file(e.what());
        }
        std::set<std::string> shards;
        if (const Json* wm = j.find("weight_map"))
            if (wm->is_object())
                for (const auto& m : wm->members())
                    if (m.second.is_string()) shards.insert(m.second.as_string());
        std::string missing;
        for (const auto& s : shards)
            if (!file_exists(folder + "/" + s)) missing += (missing.empty() ? "" : ", ") + s;
        if (!missing.empty()) fail(IMP_ERROR_FILE_NOT_FOUND, index + ": shard files missing: " + missing);
        for (const auto& s : shards) out.emplace_back(new SafetensorsFile(folder + "/" + s));
        return out;
    }
    if (file_exists(single)) {
        out.emplace_back(new SafetensorsFile(single));
        return out;
    }
    fail(IMP_ERROR_FILE_NOT_FOUND, "no model.safetensors (or model.safetensors.index.json) in " + folder);
}

void save_safetensors(const std::string& path, const std::vector<HostTensor>& tensors, const Json& metadata) {
    std::vector<const HostTensor*> order;
    for (const auto& t : tensors) order.push_back(&t);
    std::sort(order.begin(), order.end(), [](const HostTensor* a, const HostTensor* b) { return a->name < b->name; });
    Json header = Json::object();
    if (metadata.is_object() && metadata.size()) header["__metadata__"] = metadata;
    int64_t offset = 0;
    for (const HostTensor* t : order) {
        Json e = Json::object();
        e["dtype"] = t->dtype;
        e["shape"] = Json::array_of(t->shape);
        e["data_offsets"] = Json::array_of(std::vector<int64_t>{offset, offset + (int64_t)t->data.size()});
        header[t->name] = e;
        offset += (int64_t)t->data.size();
    }
    std::string h = header.dump();
    while (h.size() % 8) h.push_back(' ');
    const std::string tmp = path + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) fail(IMP_ERROR_FILE_NOT_FOUND, path + ": cannot write");
    const uint64_t hlen = h.size();
    bool ok = fwrite(&hlen, 8, 1, f) == 1 && fwrite(h.data(), 1, h.size(), f) == h.size();
    for (const HostTensor* t : order)
        if (ok && !t->data.empty()) ok = fwrite(t->data.data(), 1, t->data.size(), f) == t->data.size();
    ok = (fclose(f) == 0) && ok;
    if (!ok || rename(tmp.c_str(), path.c_str()) != 0) fail(IMP_ERROR_INTERNAL, path + ": write failed");
}

// ------------------------------------------------------------------------------------ binding
void check_checkpoint(const std::vector<std::pair<std::string, TensorSpec>>& expected,
                      const std::map<std::string, FoundTensor>& found, const std::vector<std::string>& ignored,
                      const std::string& where) {
    std::vector<std::string> missing, unexpected, wrong_shape, wrong_type;
    std::set<std::string> names;
    for (const auto& e : expected) {
        names.insert(e.first);
        auto it = found.find(e.first);
        if (it == found.end()) {
            if (!e.second.optional) missing.push_back(e.first);
            continue;
        }
        if (it->second.shape != e.second.shape)
            wrong_shape.push_back(e.first + ": expected " + shape_str(e.second.shape) + ", found " + shape_str(it->second.shape));
        const std::string& dt = it->second.dtype;
        const bool floating = dt == "F32" || dt == "BF16" || dt == "F16" || dt == "F64";
        const bool integer = dt == "I32" || dt == "I64" || dt == "I16" || dt == "I8" || dt == "U8";
        if (e.second.role == "int_table" ? !integer : !floating)
            wrong_type.push_back(e.first + ": a " + e.second.role + " must be stored as " +
                                 (e.second.role == "int_table" ? "an integer type" : "a floating-point type") + ", found " + dt);
    }
    for (const auto& f : found)
        if (!names.count(f.first) && std::find(ignored.begin(), ignored.end(), f.first) == ignored.end())
            unexpected.push_back(f.first);
    if (missing.empty() && unexpected.empty() && wrong_shape.empty() && wrong_type.empty()) return;
    auto join = [](std::vector<std::string> v, const char* sep) {
        std::sort(v.begin(), v.end());
        std::string s;
        for (const auto& x : v) s += (s.empty() ? "" : sep) + x;
        return s;
    };
    std::string msg = "checkpoint " + where + " does not match the model:";
    if (!missing.empty()) msg += "\n  missing tensors (" + std::to_string(missing.size()) + "): " + join(missing, ", ");
    if (!unexpected.empty()) msg += "\n  unexpected tensors (" + std::to_string(unexpected.size()) + "): " + join(unexpected, ", ");
    if (!wrong_shape.empty()) msg += "\n  wrong shapes (" + std::to_string(wrong_shape.size()) + "): " + join(wrong_shape, "; ");
    if (!wrong_type.empty()) msg += "\n  wrong element types (" + std::to_string(wrong_type.size()) + "): " + join(wrong_type, "; ");
    fail(IMP_ERROR_INVALID_MODEL, msg);
}

int device_dtype(const std::string& stored, const std::string& role, int compute_dtype) {
    if (role == "int_table") return I32;
    if (compute_dtype == F32) return F32;
    if (stored == "F32" || stored == "F64") return F32;
    return BF16;
}

// ---------------------------------------------------------------------------------- placement
namespace {
inline float bf16_to_float(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline uint16_t float_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);   // NaN stays NaN
    u += 0x7fffu + ((u >> 16) & 1u);                                            // round to nearest even
    return (uint16_t)(u >> 16);
}
inline float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// Host conversion for the stored types the device kernels do not read (F16, F64, small integers).
std::vector<uint8_t> convert_on_host(const StoredTensor& src, int target) {
    int64_t n = 1;
    for (int64_t d : src.shape) n *= d;
    std::vector<uint8_t> out((size_t)n * elem_size(target));
    auto value = [&](int64_t i) -> double {
        const uint8_t* p = src.data;
        if (src.dtype == "F16") return half_to_float(((const uint16_t*)p)[i]);
        if (src.dtype == "BF16") return bf16_to_float(((const uint16_t*)p)[i]);
        if (src.dtype == "F32") return ((const float*)p)[i];
        if (src.dtype == "F64") return ((const double*)p)[i];
        if (src.dtype == "I64") return (double)((const int64_t*)p)[i];
        if (src.dtype == "I32") return ((const int32_t*)p)[i];
        if (src.dtype == "I16") return ((const int16_t*)p)[i];
        if (src.dtype == "I8") return ((const int8_t*)p)[i];
        return p[i];
    };
    for (int64_t i = 0; i < n; ++i) {
        const double v = value(i);
        if (target == F32) ((float*)out.data())[i] = (float)v;
        else if (target == BF16) ((uint16_t*)out.data())[i] = float_to_bf16((float)v);
        else ((int32_t*)out.data())[i] = (int32_t)v;
    }
    return out;
}
}  // namespace

Tensor place_tensor(const StoredTensor& src, const std::string& role, int compute_dtype, WeightStore& store,
                    cudaStream_t stream) {
    const int target = device_dtype(src.dtype, role, compute_dtype);
    Tensor dst = store.alloc(target, src.shape);
    const int64_t n = numel(dst);
    if (n == 0) return dst;
    const bool same = (src.dtype == "F32" && target == F32) || (src.dtype == "BF16" && target == BF16) ||
                      (src.dtype == "I32" && target == I32);
    if (same) {
        IMP_CUDA(cudaMemcpyAsync(dst.data, src.data, src.bytes, cudaMemcpyHostToDevice, stream));
    } else if ((src.dtype == "BF16" && target == F32) || (src.dtype == "F32" && target == BF16)) {
        // widen (or round) on the device: the host copy stays in its stored type
        DeviceBuffer tmp(src.bytes);
        IMP_CUDA(cudaMemcpyAsync(tmp.data(), src.data, src.bytes, cudaMemcpyHostToDevice, stream));
        check_launch(imp_cast(dst.data, target, tmp.data(), src.dtype == "F32" ? F32 : BF16, n, stream), "cast");
        IMP_CUDA(cudaStreamSynchronize(stream));
    } else {
        std::vector<uint8_t> host = convert_on_host(src, target);
        IMP_CUDA(cudaMemcpyAsync(dst.data, host.data(), host.size(), cudaMemcpyHostToDevice, stream));
        IMP_CUDA(cudaStreamSynchronize(stream));
    }
    return dst;
}

Tensor place_device_tensor(const Tensor& src, const std::string& role, int compute_dtype, WeightStore& store,
                           cudaStream_t stream) {
    const char* stored = src.dtype == F32 ? "F32" : src.dtype == BF16 ? "BF16" : "I32";
    const int target = device_dtype(stored, role, compute_dtype);
    std::vector<int64_t> shape(src.shape, src.shape + src.ndim);
    Tensor dst = store.alloc(target, shape);
    const int64_t n = numel(dst);
    if (n == 0) return dst;
    if (target == src.dtype) {
        IMP_CUDA(cudaMemcpyAsync(dst.data, src.data, (size_t)n * elem_size(target), cudaMemcpyDeviceToDevice, stream));
    } else if (target != I32 && src.dtype != I32) {
        check_launch(imp_cast(dst.data, target, src.data, src.dtype, n, stream), "cast");
    } else {
        fail(IMP_ERROR_INVALID_ARG, std::string("a ") + role + " cannot be made from " + dtype_name(src.dtype) + " data");
    }
    return dst;
}

// ------------------------------------------------------------------------------ random weights
uint64_t tensor_seed(int64_t seed, const std::string& name) {
    uint64_t h = 0xcbf29ce484222325ull ^ ((uint64_t)seed * 0x9E3779B97F4A7C15ull);
    for (unsigned char c : name) {
        h ^= c;
        h *= 0x100000001b3ull;
    }
    h ^= h >> 29;
    h *= 0xBF58476D1CE4E5B9ull;
    h ^= h >> 32;
    return h;
}

static inline float normal_at(uint64_t tseed, uint64_t i) {
    uint64_t z = tseed + (i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    const float u1 = (float)((z >> 40) + 1) * (1.0f / 16777216.0f);          // (0, 1]
    const float u2 = (float)(z & 0xFFFFFFull) * (1.0f / 16777216.0f);        // [0, 1)
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

void random_values_host(float* out, int64_t first, int64_t n, uint64_t tseed, const std::string& init, float std,
                        float norm_std) {
    if (init == "zeros") {
        std::fill(out, out + n, 0.f);
    } else if (init == "arange_mod") {
        for (int64_t i = 0; i < n; ++i) out[i] = (float)((first + i) % 32768);
    } else if (init == "one_plus_normal") {
        for (int64_t i = 0; i < n; ++i) out[i] = 1.0f + norm_std * normal_at(tseed, (uint64_t)(first + i));
    } else {
        for (int64_t i = 0; i < n; ++i) out[i] = std * normal_at(tseed, (uint64_t)(first + i));
    }
}

Tensor random_device_tensor(const std::string& name, const TensorSpec& spec, int64_t seed, float std, float norm_std,
                            const std::string& stored_dtype, int compute_dtype, WeightStore& store, cudaStream_t stream) {
    // values are made in the stored type's precision first, as a checkpoint would hold them
    const int target = device_dtype(stored_dtype, spec.role, compute_dtype);
    Tensor dst = store.alloc(target, spec.shape);
    const int64_t n = numel(dst);
    if (n == 0) return dst;
    const int mode = spec.role == "int_table" || spec.init == "arange_mod" ? 3
                     : spec.init == "zeros"                                 ? 2
                     : spec.init == "one_plus_normal"                       ? 1
                                                                            : 0;
    const int round_bf16 = (stored_dtype == "BF16" || stored_dtype == "bfloat16") ? 1 : 0;
    check_launch(imp_random_fill(dst.data, target, n, tensor_seed(seed, name), mode, std, norm_std, round_bf16, stream),
                 "random_fill");
    return dst;
}

void write_random_model(const Json& config, const ModelPlan& plan, const std::string& folder, int64_t seed, float std,
                        float norm_std, const std::string& store_dtype) {
    mkdir(folder.c_str(), 0777);
    {
        std::ofstream f(folder + "/config.json");
        if (!f) fail(IMP_ERROR_FILE_NOT_FOUND, folder + "/config.json: cannot write");
        f << config.dump(2) << "\n";
    }
    const bool bf16 = store_dtype == "bfloat16" || store_dtype == "bf16";
    if (!bf16 && store_dtype != "float32" && store_dtype != "fp32")
        fail(IMP_ERROR_INVALID_ARG, "weights are stored as bfloat16 or float32, not '" + store_dtype + "'");
    std::vector<HostTensor> tensors;
    for (const auto& e : plan.expected_tensors()) {
        HostTensor t;
        t.name = e.first;
        t.shape = e.second.shape;
        const int64_t n = e.second.numel();
        const bool ints = e.second.role == "int_table";
        t.dtype = ints ? "I32" : bf16 ? "BF16" : "F32";
        t.data.resize((size_t)n * (ints || !bf16 ? 4 : 2));
        const uint64_t ts = tensor_seed(seed, e.first);
        const std::string init = ints ? "arange_mod" : e.second.init;
        const int n_threads = n > (1 << 20) ? (int)std::min<int64_t>(16, std::max(1u, std::thread::hardware_concurrency())) : 1;
        std::vector<std::thread> pool;
        const int64_t per = (n + n_threads - 1) / n_threads;
        for (int w = 0; w < n_threads; ++w) {
            const int64_t lo = w * per, hi = std::min(n, lo + per);
            if (lo >= hi) break;
            auto work = [&, lo, hi] {
                std::vector<float> buf((size_t)std::min<int64_t>(hi - lo, 1 << 16));
                for (int64_t a = lo; a < hi; a += (int64_t)buf.size()) {
                    const int64_t m = std::min<int64_t>((int64_t)buf.size(), hi - a);
                    random_values_host(buf.data(), a, m, ts, init, std, norm_std);
                    for (int64_t i = 0; i < m; ++i) {
                        if (ints) ((int32_t*)t.data.data())[a + i] = (int32_t)buf[(size_t)i];
                        else if (bf16) ((uint16_t*)t.data.data())[a + i] = float_to_bf16(buf[(size_t)i]);
                        else ((float*)t.data.data())[a + i] = buf[(size_t)i];
                    }
                }
            };
            if (n_threads == 1) work();
            else pool.emplace_back(work);
        }
        for (auto& th : pool) th.join();
        tensors.push_back(std::move(t));
    }
    Json meta = Json::object();
    meta["format"] = "pt";
    meta["seed"] = std::to_string(seed);
    meta["std"] = std::to_string(std);
    save_safetensors(folder + "/model.safetensors", tensors, meta);
}

}  // namespace imp
