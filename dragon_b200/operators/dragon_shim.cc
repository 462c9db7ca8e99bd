// Implementation of the Dragon-core stand-in declared in dragon_shim.h.
#include "dragon_shim.h"

#include <cuda_runtime.h>

#include <mutex>

namespace dragon {

#define SHIM_CUDA_CHECK(expr)                                                            \
  do {                                                                                   \
    cudaError_t e__ = (expr);                                                            \
    CHECK(e__ == cudaSuccess) << "\nCUDA: " << cudaGetErrorString(e__) << " in " #expr;  \
  } while (0)

// ---- OperatorDef wire form -------------------------------------------------------

OperatorDef OperatorDef::Parse(const string& text) {
  OperatorDef def;
  std::istringstream lines(text);
  string line;
  while (std::getline(lines, line)) {
    if (line.empty()) continue;
    std::istringstream in(line);
    string key;
    in >> key;
    if (key == "type") {
      in >> def.type;
    } else if (key == "name") {
      in >> def.name;
    } else if (key == "input") {
      string v;
      in >> v;
      def.input.push_back(v);
    } else if (key == "output") {
      string v;
      in >> v;
      def.output.push_back(v);
    } else if (key == "device") {
      in >> def.device_option.device_type >> def.device_option.device_id;
    } else if (key == "arg_i" || key == "arg_s" || key == "arg_ints" || key == "arg_f" || key == "arg_floats") {
      Argument a;
      in >> a.name;
      if (key == "arg_i") {
        in >> a.i;
      } else if (key == "arg_f") {
        in >> a.f;
      } else if (key == "arg_s") {
        in >> std::ws;
        std::getline(in, a.s);
      } else if (key == "arg_floats") {
        double v;
        while (in >> v) a.floats.push_back(v);
      } else {
        int64_t v;
        while (in >> v) a.ints.push_back(v);
      }
      def.arg.push_back(a);
    } else {
      DRAGON_FATAL << "Unknown key in operator definition: " << key;
    }
  }
  return def;
}

// ---- Tensor ------------------------------------------------------------------------

Tensor::~Tensor() {
  if (data_ && !external_) {
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(device_id_);
    cudaFree(data_);
    cudaSetDevice(prev);
  }
}

void Tensor::ShareExternal(void* ptr, const vec64_t& dims, DType dtype, int device_id, size_t capacity_bytes) {
  CHECK(!data_ || external_) << "\nTensor(" << name_ << ") already owns memory.";
  data_ = ptr;
  dims_ = dims;
  dtype_ = dtype;
  device_id_ = device_id;
  capacity_ = capacity_bytes;
  external_ = true;
}

void Tensor::EnsureCapacity(DType dtype) {
  const size_t need = static_cast<size_t>(count()) * dtype_size(dtype);
  if (external_) {
    CHECK(dtype == dtype_) << "\nTensor(" << name_ << ") holds external " << dtype_name(dtype_)
                           << " memory, while requesting " << dtype_name(dtype) << ".";
    CHECK(need <= capacity_) << "\nTensor(" << name_ << ") holds " << capacity_
                             << " external bytes, while requesting " << need << ".";
    return;
  }
  dtype_ = dtype;
  if (need <= capacity_ && data_) return;
  // Plain cudaMalloc rounded up to 512 bytes, one allocation per tensor
  // (core/context_cuda.h:172-177); memory is kept across runs.
  int dev = 0;
  SHIM_CUDA_CHECK(cudaGetDevice(&dev));
  if (data_) SHIM_CUDA_CHECK(cudaFree(data_));
  capacity_ = (need + 511) / 512 * 512;
  if (capacity_ == 0) capacity_ = 512;
  SHIM_CUDA_CHECK(cudaMalloc(&data_, capacity_));
  device_id_ = dev;
}

// ---- Workspace ---------------------------------------------------------------------

Workspace::~Workspace() {
  operators_.clear();
  tensors_.clear();
}

Tensor* Workspace::CreateTensor(const string& name) {
  auto it = tensors_.find(name);
  if (it != tensors_.end()) return it->second.get();
  auto* t = new Tensor(name);
  tensors_[name].reset(t);
  return t;
}

Tensor* Workspace::GetTensor(const string& name) const {
  auto it = tensors_.find(name);
  CHECK(it != tensors_.end()) << "\nTensor(" << name << ") does not exist.";
  return it->second.get();
}

void Workspace::RunOperator(const OperatorDef& def, int stream, bool sync) {
  string cache_key;
  if (!def.arg.empty() && def.arg.back().name == "cache_key") cache_key = def.arg.back().s;
  if (cache_key.empty()) {
    std::unique_ptr<OperatorBase> op(OperatorBase::New(def, this));
    op->Run(stream, sync);
    return;
  }
  auto it = operators_.find(cache_key);
  if (it == operators_.end()) {
    operators_[cache_key].reset(OperatorBase::New(def, this));
    it = operators_.find(cache_key);
  }
  it->second->DeriveFrom(def)->Run(stream, sync);
}

// ---- CUDAContext -----------------------------------------------------------------------

namespace {
struct DeviceObjects {
  std::map<int, cudaStream_t> streams;                  // by stream id
  std::map<int, std::unique_ptr<Workspace>> workspaces;  // by stream id
  cudaStream_t external = nullptr;
  bool has_external = false;
};
std::mutex g_objects_mutex;
std::map<int, DeviceObjects>& objects() {
  static std::map<int, DeviceObjects> o;
  return o;
}
}  // namespace

void CUDAContext::SetExternalStream(int device_id, void* stream) {
  std::lock_guard<std::mutex> lock(g_objects_mutex);
  DeviceObjects& d = objects()[device_id];
  d.external = static_cast<cudaStream_t>(stream);
  d.has_external = true;
}

void CUDAContext::SwitchToDevice(int stream) {
  SHIM_CUDA_CHECK(cudaSetDevice(device_id_));
  stream_id_ = stream;
}

void* CUDAContext::cuda_stream() {
  std::lock_guard<std::mutex> lock(g_objects_mutex);
  DeviceObjects& d = objects()[device_id_];
  if (stream_id_ == 0 && d.has_external) return d.external;
  auto it = d.streams.find(stream_id_);
  if (it == d.streams.end()) {
    cudaStream_t s = nullptr;
    SHIM_CUDA_CHECK(cudaSetDevice(device_id_));
    SHIM_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    it = d.streams.emplace(stream_id_, s).first;
  }
  return it->second;
}

void CUDAContext::FinishDeviceComputation() {
  SHIM_CUDA_CHECK(cudaStreamSynchronize(static_cast<cudaStream_t>(cuda_stream())));
}

Workspace* CUDAContext::workspace() {
  std::lock_guard<std::mutex> lock(g_objects_mutex);
  auto& slot = objects()[device_id_].workspaces[stream_id_];
  if (!slot) slot.reset(new Workspace());
  return slot.get();
}

// ---- OperatorBase ------------------------------------------------------------------------

OperatorBase::OperatorBase(const OperatorDef& def, Workspace* ws) : def_(def), ws_(ws) {
  for (const Argument& a : def_.arg) {
    CHECK(args_.count(a.name) == 0) << "\nDuplicated argument: " << a.name;
    args_[a.name] = &a;
  }
  for (const string& name : def_.input) inputs_.push_back(ws->GetTensor(name));
  for (const string& name : def_.output) outputs_.push_back(ws->CreateTensor(name));
}

OperatorBase* OperatorBase::DeriveFrom(const OperatorDef& def) {
  inputs_.resize(def.input.size());
  outputs_.resize(def.output.size());
  for (size_t i = 0; i < inputs_.size(); ++i) inputs_[i] = ws_->GetTensor(def.input[i]);
  for (size_t i = 0; i < outputs_.size(); ++i) outputs_[i] = ws_->CreateTensor(def.output[i]);
  return this;
}

Tensor& OperatorBase::Input(int i) {
  CHECK(i >= 0 && i < InputSize()) << "\nInput index " << i << " is out of range.";
  return *inputs_[i];
}

Tensor* OperatorBase::Output(int i) {
  if (i < 0) i += OutputSize();  // Output(-1) is the last output, as in the reference
  CHECK(i >= 0 && i < OutputSize()) << "\nOutput index " << i << " is out of range.";
  return outputs_[i];
}

const Argument* OperatorBase::FindArg(const string& name) const {
  auto it = args_.find(name);
  return it == args_.end() ? nullptr : it->second;
}

OperatorBase* OperatorBase::New(const OperatorDef& def, Workspace* ws) {
  CHECK(def.device_option.device_type == PROTO_CUDA)
      << "\nOnly the CUDA registry exists in this library (device_type " << def.device_option.device_type << ").";
  CHECK(CUDAOperatorRegistry()->Has(def.type)) << "\nOperator type is not registered: " << def.type;
  return CUDAOperatorRegistry()->Create(def.type, def, ws);
}

// ---- registry / schema -------------------------------------------------------------------

void OperatorRegistry::Register(const string& key, Creator creator) {
  CHECK(creators_.count(key) == 0) << "\nKey(" << key << ") has already registered.";
  creators_[key] = creator;
}

OperatorBase* OperatorRegistry::Create(const string& key, const OperatorDef& def, Workspace* ws) const {
  auto it = creators_.find(key);
  CHECK(it != creators_.end()) << "\nKey(" << key << ") is not registered.";
  return it->second(def, ws);
}

vector<string> OperatorRegistry::Keys() const {
  vector<string> keys;
  for (const auto& kv : creators_) keys.push_back(kv.first);
  return keys;
}

OperatorRegistry* CUDAOperatorRegistry() {
  static OperatorRegistry* registry = new OperatorRegistry();
  return registry;
}

namespace {
std::map<string, OpSchema>& schemas() {
  static std::map<string, OpSchema> s;
  return s;
}
}  // namespace

OpSchema& OpSchema::NewSchema(const string& op_type) {
  CHECK(schemas().count(op_type) == 0) << "\nOpSchema(" << op_type << ") has registered.";
  return schemas()[op_type];
}

const OpSchema* OpSchema::Find(const string& op_type) {
  auto it = schemas().find(op_type);
  return it == schemas().end() ? nullptr : &it->second;
}

}  // namespace dragon
