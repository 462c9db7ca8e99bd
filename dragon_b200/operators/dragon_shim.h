// A stand-in for the slice of Dragon's core that `CollectiveOp` touches, so the
// operator source in this directory compiles and runs without a Dragon build:
// OperatorDef / Argument (plain structs instead of protobuf messages), Tensor,
// Workspace, CUDAContext, OperatorBase / Operator<Context>, the operator
// registry and its macros, dtype dispatch, LOG(FATAL) / CHECK.
//
// Names, argument meaning and error behaviour follow Dragon
// (dragon/core/operator.h:214-219,318-322,429-450; core/registry.h:23-115;
// core/tensor.h:291-345; core/workspace.cc:73-94; proto/dragon.proto:56-96).
// Only what the collective path needs exists here; this is not a framework.
// One difference: a fatal error throws dragon::FatalError (which the C entry
// points of this library turn into a status code) instead of calling abort().
#ifndef DRAGON_B200_OPERATORS_DRAGON_SHIM_H_
#define DRAGON_B200_OPERATORS_DRAGON_SHIM_H_

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace dragon {

using std::string;
using std::vector;
typedef vector<int64_t> vec64_t;

// ---- logging ---------------------------------------------------------------

struct FatalError : std::runtime_error {
  explicit FatalError(const string& what) : std::runtime_error(what) {}
};

class FatalMessage {
 public:
  FatalMessage(const char* file, int line) { stream_ << "FATAL " << file << ":" << line << "] "; }
  [[noreturn]] ~FatalMessage() noexcept(false) { throw FatalError(stream_.str()); }
  std::ostringstream& stream() { return stream_; }

 private:
  std::ostringstream stream_;
};

#define DRAGON_FATAL ::dragon::FatalMessage(__FILE__, __LINE__).stream()
#define LOG_FATAL DRAGON_FATAL
#define CHECK(cond) \
  if (!(cond)) DRAGON_FATAL << "Check failed: " #cond " "
#define CHECK_EQ(a, b) CHECK((a) == (b))
#define CHECK_LT(a, b) CHECK((a) < (b))

// ---- dtypes ------------------------------------------------------------------

struct float16 { uint16_t x; };
struct bfloat16 { uint16_t x; };

// The reference's dtypes::Numerical list (dragon/core/types.h:69), by name.
enum class DType : int { kUInt8 = 0, kInt8, kInt32, kInt64, kFloat16, kBFloat16, kFloat32, kFloat64, kUnknown };

inline size_t dtype_size(DType t) {
  static const size_t s[] = {1, 1, 4, 8, 2, 2, 4, 8, 0};
  return s[static_cast<int>(t)];
}
inline const char* dtype_name(DType t) {
  static const char* n[] = {"uint8", "int8", "int32", "int64", "float16", "bfloat16", "float32", "float64", "unknown"};
  return n[static_cast<int>(t)];
}
inline DType dtype_from_name(const string& s) {
  for (int i = 0; i < 8; ++i)
    if (s == dtype_name(static_cast<DType>(i))) return static_cast<DType>(i);
  return DType::kUnknown;
}
template <typename T> struct DTypeOf;
template <> struct DTypeOf<uint8_t> { static constexpr DType value = DType::kUInt8; };
template <> struct DTypeOf<int8_t> { static constexpr DType value = DType::kInt8; };
template <> struct DTypeOf<int> { static constexpr DType value = DType::kInt32; };
template <> struct DTypeOf<int64_t> { static constexpr DType value = DType::kInt64; };
template <> struct DTypeOf<float16> { static constexpr DType value = DType::kFloat16; };
template <> struct DTypeOf<bfloat16> { static constexpr DType value = DType::kBFloat16; };
template <> struct DTypeOf<float> { static constexpr DType value = DType::kFloat32; };
template <> struct DTypeOf<double> { static constexpr DType value = DType::kFloat64; };

// ---- operator definition (dragon.proto OperatorDef / Argument / DeviceOption) ---

struct Argument {
  string name;
  int64_t i = 0;
  double f = 0;
  string s;
  vector<int64_t> ints;
  vector<double> floats;
  vector<string> strings;
};

enum DeviceTypeProto { PROTO_CPU = 0, PROTO_CUDA = 1 };

struct DeviceOption {
  int device_type = PROTO_CPU;
  int device_id = 0;
};

struct OperatorDef {
  string name, type;
  vector<string> input, output;
  vector<Argument> arg;
  DeviceOption device_option;

  // Line-oriented wire form used by the C entry points (the reference ships a
  // serialised protobuf through pybind at the same place):
  //   type Collective | name OpName | input X | output Y | device 1 0 |
  //   arg_i name 3 | arg_f name 0.5 | arg_s name TEXT | arg_ints name 0 1 2 | arg_floats name 1 0.5
  static OperatorDef Parse(const string& text);
};

// ---- tensors ---------------------------------------------------------------------

class CUDAContext;
// Tag for host-side access, as in data<T, CPUContext>().  A tensor fed with
// device id -1 holds host memory (the hyper tensors of the update operators).
class CPUContext {};

class Tensor {
 public:
  explicit Tensor(const string& name = "") : name_(name) {}
  ~Tensor();
  Tensor(const Tensor&) = delete;
  Tensor& operator=(const Tensor&) = delete;

  const string& name() const { return name_; }
  const vec64_t& dims() const { return dims_; }
  int64_t count() const {
    int64_t n = 1;
    for (auto d : dims_) n *= d;
    return n;
  }
  int64_t dim(int i) const { return dims_[i]; }
  DType dtype() const { return dtype_; }
  size_t nbytes() const { return static_cast<size_t>(count()) * dtype_size(dtype_); }
  int device_id() const { return device_id_; }

  Tensor* Reshape(const vec64_t& dims) {
    dims_ = dims;
    return this;
  }
  Tensor* ReshapeLike(const Tensor& other) { return Reshape(other.dims_); }

  // Points the tensor at memory owned by someone else (a torch tensor, a
  // Dragon tensor).  Such a tensor is never reallocated: a size or type
  // mismatch at mutable_data() is fatal.
  void ShareExternal(void* ptr, const vec64_t& dims, DType dtype, int device_id, size_t capacity_bytes);

  template <typename T, class Context>
  const T* data() const {
    CHECK(dtype_ == DTypeOf<T>::value) << "\nThe type of Tensor(" << name_ << ") is " << dtype_name(dtype_)
                                       << ", while requesting " << dtype_name(DTypeOf<T>::value) << ".";
    CHECK(data_ != nullptr || count() == 0) << "\nRead Tensor(" << name_ << ") with no memory.";
    return static_cast<const T*>(data_);
  }

  template <typename T, class Context>
  T* mutable_data() {
    EnsureCapacity(DTypeOf<T>::value);
    return static_cast<T*>(data_);
  }

  const void* raw_data() const { return data_; }
  void* raw_mutable_data(DType dtype) {
    EnsureCapacity(dtype);
    return data_;
  }

 private:
  void EnsureCapacity(DType dtype);

  string name_;
  vec64_t dims_;
  DType dtype_ = DType::kUnknown;
  void* data_ = nullptr;
  size_t capacity_ = 0;
  bool external_ = false;
  int device_id_ = 0;
};

// ---- workspace ----------------------------------------------------------------------

class OperatorBase;

class Workspace {
 public:
  Workspace() = default;
  ~Workspace();

  Tensor* CreateTensor(const string& name);
  Tensor* GetTensor(const string& name) const;  // fatal if absent (core/operator.cc:18-22)
  bool HasTensor(const string& name) const { return tensors_.count(name) != 0; }
  void RemoveTensor(const string& name) { tensors_.erase(name); }

  // Runs an operator; an OperatorDef whose last argument is `cache_key`
  // reuses the operator instance created for that key (workspace.cc:76-92).
  void RunOperator(const OperatorDef& def, int stream = 0, bool sync = false);

 private:
  std::map<string, std::unique_ptr<Tensor>> tensors_;
  std::map<string, std::unique_ptr<OperatorBase>> operators_;
};

// ---- CUDA context ----------------------------------------------------------------------

// Streams are kept per (device, stream id) for the life of the process, like
// the thread-local CUDAObjects of the reference (core/context_cuda.cc:35-46).
// Stream id 0 with an externally supplied stream lets a host framework (torch
// in the tests) put the work on its own stream.
class CUDAContext {
 public:
  explicit CUDAContext(const DeviceOption& opt) : device_id_(opt.device_id) {}
  void SwitchToDevice(int stream);
  void* cuda_stream();                 // cudaStream_t
  void FinishDeviceComputation();      // cudaStreamSynchronize
  int device() const { return device_id_; }
  Workspace* workspace();              // per (device, stream) scratch workspace

  static void SetExternalStream(int device_id, void* stream);  // stream id 0 of that device

 private:
  int device_id_ = 0, stream_id_ = 0;
};

// ---- operators ---------------------------------------------------------------------------

class OperatorBase {
 public:
  OperatorBase(const OperatorDef& def, Workspace* ws);
  virtual ~OperatorBase() {}

  virtual void Run(int stream = 0, bool sync = false) = 0;

  // Re-points a cached operator at the tensors of a new definition
  // (core/operator.cc:100-115): inputs and outputs may differ every run.
  OperatorBase* DeriveFrom(const OperatorDef& def);

  Tensor& Input(int i);
  Tensor* Output(int i);
  int InputSize() const { return static_cast<int>(inputs_.size()); }
  int OutputSize() const { return static_cast<int>(outputs_.size()); }
  const string& type() const { return def_.type; }
  const string& name() const { return def_.name; }
  const OperatorDef& def() const { return def_; }
  Workspace* workspace() const { return ws_; }

  template <typename T> T GetArgument(const string& name, const T& dflt);
  template <typename T> T GetArgument(const string& name);

  static OperatorBase* New(const OperatorDef& def, Workspace* ws);

 protected:
  const Argument* FindArg(const string& name) const;
  OperatorDef def_;
  Workspace* ws_;
  vector<Tensor*> inputs_, outputs_;
  std::map<string, const Argument*> args_;
};

#define OP_SINGLE_ARG(type, name, default) OperatorBase::GetArgument<type>(name, (default))
#define OP_REPEATED_ARG(type, name) OperatorBase::GetArgument<vector<type>>(name)
#define USE_OPERATOR_FUNCTIONS   \
  using OperatorBase::Input;     \
  using OperatorBase::Output;    \
  using OperatorBase::InputSize; \
  using OperatorBase::OutputSize

template <class Context>
class Operator : public OperatorBase {
 public:
  Operator(const OperatorDef& def, Workspace* ws) : OperatorBase(def, ws), ctx_(def.device_option) {}

  // Setup; switch to the device and stream; run; optionally wait
  // (core/operator.h:214-219).  The op never synchronises on its own.
  void Run(int stream = 0, bool sync = false) final {
    ctx()->SwitchToDevice(stream);
    RunOnDevice();
    if (sync) ctx()->FinishDeviceComputation();
  }
  virtual void RunOnDevice() = 0;
  Context* ctx() { return &ctx_; }

 protected:
  Context ctx_;
};

// Registry keyed by the operator type string; registering a key twice is
// fatal (core/registry.h:44-48), so a replacement operator takes the place of
// the built-in registration line, it cannot sit beside it.
class OperatorRegistry {
 public:
  typedef std::function<OperatorBase*(const OperatorDef&, Workspace*)> Creator;
  void Register(const string& key, Creator creator);
  bool Has(const string& key) const { return creators_.count(key) != 0; }
  OperatorBase* Create(const string& key, const OperatorDef& def, Workspace* ws) const;
  vector<string> Keys() const;

 private:
  std::unordered_map<string, Creator> creators_;
};

OperatorRegistry* CUDAOperatorRegistry();

struct OperatorRegisterer {
  OperatorRegisterer(OperatorRegistry* registry, const string& key, OperatorRegistry::Creator creator) {
    registry->Register(key, creator);
  }
};

#define DRAGON_CONCAT_(a, b) a##b
#define DRAGON_CONCAT(a, b) DRAGON_CONCAT_(a, b)
#define REGISTER_CUDA_OPERATOR(name, ...)                                                         \
  static ::dragon::OperatorRegisterer DRAGON_CONCAT(g_cuda_operator_##name##_, __LINE__)(         \
      ::dragon::CUDAOperatorRegistry(), #name,                                                    \
      [](const ::dragon::OperatorDef& def, ::dragon::Workspace* ws) -> ::dragon::OperatorBase* { \
        return new __VA_ARGS__(def, ws);                                                          \
      })
#define DEPLOY_CUDA_OPERATOR(name) REGISTER_CUDA_OPERATOR(name, name##Op<CUDAContext>)

// Schema: only the in-place rule is kept (core/operator_schema.h:76-101).
class OpSchema {
 public:
  OpSchema& AllowInplace(std::function<bool(int, int)> fn) {
    inplace_ = fn;
    return *this;
  }
  bool CheckInplace(int in, int out) const { return inplace_ ? inplace_(in, out) : false; }
  static OpSchema& NewSchema(const string& op_type);  // fatal on a duplicate
  static const OpSchema* Find(const string& op_type);

 private:
  std::function<bool(int, int)> inplace_;
};
#define OPERATOR_SCHEMA(name) \
  static ::dragon::OpSchema* DRAGON_CONCAT(g_schema_##name##_, __LINE__) = &::dragon::OpSchema::NewSchema(#name)

// Calls op->DoRunWithType<T>() for the tensor's element type over the
// Numerical list; any other type is fatal and names the op.
namespace dtypes {
struct Numerical {};
struct Floating {};  // float16, bfloat16, float32, float64 (dragon/core/types.h)
}
template <class Types> struct DispatchHelper;
template <>
struct DispatchHelper<dtypes::Numerical> {
  template <class Op>
  static void Call(Op* op, const Tensor& x) {
    switch (x.dtype()) {
      case DType::kUInt8: return op->template DoRunWithType<uint8_t>();
      case DType::kInt8: return op->template DoRunWithType<int8_t>();
      case DType::kInt32: return op->template DoRunWithType<int>();
      case DType::kInt64: return op->template DoRunWithType<int64_t>();
      case DType::kFloat16: return op->template DoRunWithType<float16>();
      case DType::kBFloat16: return op->template DoRunWithType<bfloat16>();
      case DType::kFloat32: return op->template DoRunWithType<float>();
      case DType::kFloat64: return op->template DoRunWithType<double>();
      default:
        DRAGON_FATAL << "Unsupported type: " << dtype_name(x.dtype()) << "\n<" << op->type()
                     << "Op> supports the numerical types only.";
    }
  }
};

template <>
struct DispatchHelper<dtypes::Floating> {
  template <class Op>
  static void Call(Op* op, const Tensor& x) {
    switch (x.dtype()) {
      case DType::kFloat16: return op->template DoRunWithType<float16>();
      case DType::kBFloat16: return op->template DoRunWithType<bfloat16>();
      case DType::kFloat32: return op->template DoRunWithType<float>();
      case DType::kFloat64: return op->template DoRunWithType<double>();
      default:
        DRAGON_FATAL << "Unsupported type: " << dtype_name(x.dtype()) << "\n<" << op->type()
                     << "Op> supports the floating types only.";
    }
  }
};

// ---- argument access ------------------------------------------------------------------------

template <> inline int64_t OperatorBase::GetArgument<int64_t>(const string& name, const int64_t& dflt) {
  const Argument* a = FindArg(name);
  return a ? a->i : dflt;
}
template <> inline string OperatorBase::GetArgument<string>(const string& name, const string& dflt) {
  const Argument* a = FindArg(name);
  return a ? a->s : dflt;
}
template <> inline vector<int64_t> OperatorBase::GetArgument<vector<int64_t>>(const string& name) {
  const Argument* a = FindArg(name);
  return a ? a->ints : vector<int64_t>();
}
template <> inline float OperatorBase::GetArgument<float>(const string& name, const float& dflt) {
  const Argument* a = FindArg(name);
  return a ? static_cast<float>(a->f) : dflt;
}
template <> inline vector<float> OperatorBase::GetArgument<vector<float>>(const string& name) {
  const Argument* a = FindArg(name);
  vector<float> out;
  if (a) out.assign(a->floats.begin(), a->floats.end());
  return out;
}

}  // namespace dragon

#endif  // DRAGON_B200_OPERATORS_DRAGON_SHIM_H_
