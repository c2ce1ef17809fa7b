// Checkpoints: the safetensors container, binding tensors to a plan by name with one error that
// lists every mismatch, element types on the device, and random weights by (seed, tensor name).
//
// Container format (as the reference parses it, src/model/safetensors_loader.cpp:469-568): an 8-byte
// little-endian header length, a JSON object that maps each tensor name to {"dtype", "shape",
// "data_offsets": [begin, end]} relative to the end of the header (plus an optional "__metadata__"
// entry), then the raw little-endian data.  A folder may also hold model.safetensors.index.json
// naming several shard files (the reference reads a single file only).
//
// The reference binds by splitting names and treats unknown or missing tensors as warnings
// (src/model/weight_map.cpp:152-336; the q/k norm tensors of this family are dropped on its
// safetensors route, :295-297).  Here a checkpoint must hold exactly the tensors the plan expects,
// with the expected shapes and kinds of element type.
//
// Element types on the device:
//   compute bfloat16: floating tensors stored in 16 bits become bfloat16, tensors stored in 32 bits
//       stay float32 (the kernels take either), integer tables become int32;
//   compute float32: every floating tensor is widened to float32.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "parts.hpp"
#include "plan.hpp"

namespace imp {

struct StoredTensor {
    std::string dtype;                // the container's name: F32, BF16, F16, F64, I32, I64, I16, I8, U8, BOOL
    std::vector<int64_t> shape;
    const uint8_t* data = nullptr;    // into the mapping
    size_t bytes = 0;
    bool floating() const { return dtype == "F32" || dtype == "BF16" || dtype == "F16" || dtype == "F64"; }
};

// A memory-mapped safetensors file.
class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path);   // throws Error(IMP_ERROR_INVALID_MODEL) on a malformed file
    ~SafetensorsFile();
    SafetensorsFile(const SafetensorsFile&) = delete;
    const std::string& path() const { return path_; }
    const std::vector<std::pair<std::string, StoredTensor>>& tensors() const { return tensors_; }
    const Json& metadata() const { return metadata_; }

private:
    std::string path_;
    void* map_ = nullptr;
    size_t size_ = 0;
    Json metadata_ = Json::object();
    std::vector<std::pair<std::string, StoredTensor>> tensors_;
};

// All safetensors files of a model folder: one model.safetensors, or the shards of the index.
std::vector<std::unique_ptr<SafetensorsFile>> open_model_files(const std::string& folder);

struct HostTensor {
    std::string name, dtype;          // container dtype name
    std::vector<int64_t> shape;
    std::vector<uint8_t> data;
};
void save_safetensors(const std::string& path, const std::vector<HostTensor>& tensors, const Json& metadata);

// Names, shapes and kinds of element type against the plan; throws one Error that lists what is
// missing, unexpected, of the wrong shape and of the wrong type.
struct FoundTensor { std::vector<int64_t> shape; std::string dtype; };
void check_checkpoint(const std::vector<std::pair<std::string, TensorSpec>>& expected,
                      const std::map<std::string, FoundTensor>& found, const std::vector<std::string>& ignored,
                      const std::string& where);

// The element type a tensor has on the device.
int device_dtype(const std::string& stored, const std::string& role, int compute_dtype);

// Copy one stored tensor to the device in the type the engine keeps it in.
Tensor place_tensor(const StoredTensor& src, const std::string& role, int compute_dtype, WeightStore& store,
                    cudaStream_t stream);
// The same for a tensor that already lives on the device (F32 / BF16 / I32 views).
Tensor place_device_tensor(const Tensor& src, const std::string& role, int compute_dtype, WeightStore& store,
                           cudaStream_t stream);

// Random weights: each tensor is a function of (seed, its name) alone.  Matrices are N(0, std), norm
// weights 1 + N(0, norm_std), integer tables index mod 2^15.  The reference fills test and bench models
// from one std::mt19937(42) stream, uniform in +-0.01 with norm weights 1.0
// (tools/imp-bench/bench_e2e.cpp:43-120).
uint64_t tensor_seed(int64_t seed, const std::string& name);
// Host: `n` values starting at element `first`, as float32.
void random_values_host(float* out, int64_t first, int64_t n, uint64_t tseed, const std::string& init, float std,
                        float norm_std);
// Device: fill a tensor of the store with the same values (rounded to its type).
Tensor random_device_tensor(const std::string& name, const TensorSpec& spec, int64_t seed, float std, float norm_std,
                            const std::string& stored_dtype, int compute_dtype, WeightStore& store, cudaStream_t stream);
void write_random_model(const Json& config, const ModelPlan& plan, const std::string& folder, int64_t seed, float std,
                        float norm_std, const std::string& store_dtype);

}  // namespace imp
