// C entry points of the operator layer, for hosts that are not C++ (the Python
// package, tests).  They play the part of Dragon's pybind module
// (dragon/modules/python/module.cc:84-119: Workspace.RunOperator) with plain C
// types.  A fatal error inside the operator layer comes back as status 1 and
// a message instead of abort().
#include <cstring>
#include <string>

#include "collective_op.h"
#include "dragon_shim.h"

using namespace dragon;

namespace {
thread_local std::string g_error;

template <typename Fn>
int guarded(Fn fn) {
  try {
    fn();
    return 0;
  } catch (const FatalError& e) {
    g_error = e.what();
    return 1;
  } catch (const std::exception& e) {
    g_error = e.what();
    return 1;
  }
}
}  // namespace

extern "C" {

const char* dragon_last_error(void) { return g_error.c_str(); }

void* dragon_workspace_create(void) { return new Workspace(); }

void dragon_workspace_destroy(void* ws) { delete static_cast<Workspace*>(ws); }

// Binds `name` to device memory owned by the caller.
int dragon_workspace_feed_external(void* ws, const char* name, void* ptr, const int64_t* dims, int ndim,
                                   const char* dtype, int device_id, int64_t capacity_bytes) {
  return guarded([&] {
    const DType t = dtype_from_name(dtype);
    CHECK(t != DType::kUnknown) << "\nUnsupported data type: " << dtype;
    static_cast<Workspace*>(ws)->CreateTensor(name)->ShareExternal(
        ptr, vec64_t(dims, dims + ndim), t, device_id, static_cast<size_t>(capacity_bytes));
  });
}

int dragon_workspace_remove_tensor(void* ws, const char* name) {
  return guarded([&] { static_cast<Workspace*>(ws)->RemoveTensor(name); });
}

// Shape, type and address of a tensor (e.g. an output the operator allocated).
int dragon_workspace_tensor_info(void* ws, const char* name, int64_t* dims, int max_dims, int* ndim,
                                 char* dtype, int dtype_len, void** ptr) {
  return guarded([&] {
    Tensor* t = static_cast<Workspace*>(ws)->GetTensor(name);
    CHECK(static_cast<int>(t->dims().size()) <= max_dims) << "\nToo many dimensions.";
    *ndim = static_cast<int>(t->dims().size());
    for (int i = 0; i < *ndim; ++i) dims[i] = t->dim(i);
    std::strncpy(dtype, dtype_name(t->dtype()), dtype_len - 1);
    dtype[dtype_len - 1] = '\0';
    *ptr = const_cast<void*>(t->raw_data());
  });
}

// Stream id 0 of `device_id` becomes `stream` (a cudaStream_t).
void dragon_set_external_stream(int device_id, void* stream) { CUDAContext::SetExternalStream(device_id, stream); }

// Runs one operator given in the line-oriented wire form (see OperatorDef::Parse).
int dragon_workspace_run_operator(void* ws, const char* def_text, int stream, int sync) {
  return guarded([&] {
    OperatorDef def = OperatorDef::Parse(def_text);
    static_cast<Workspace*>(ws)->RunOperator(def, stream, sync != 0);
  });
}

int dragon_operator_is_registered(const char* type) { return CUDAOperatorRegistry()->Has(type) ? 1 : 0; }

// 1 if registering `type` a second time is refused (it must be).
int dragon_registry_rejects_duplicate(const char* type) {
  int refused = 0;
  guarded([&] {
    try {
      CUDAOperatorRegistry()->Register(type, [](const OperatorDef&, Workspace*) -> OperatorBase* { return nullptr; });
    } catch (const FatalError&) {
      refused = 1;
    }
  });
  return refused;
}

int dragon_schema_allows_inplace(const char* type, int in, int out) {
  const OpSchema* s = OpSchema::Find(type);
  return (s && s->CheckInplace(in, out)) ? 1 : 0;
}

}  // extern "C"
