// dgn_allreduce_static: an all-reduce over several buffers that live on ONE
// device, for callers that are not allowed to allocate.
//
// Who needs it: code that runs with every byte of device memory already
// handed out (a framework whose workspace planner owns the whole pool), code
// on a serving path that must never take the allocator's device-wide
// synchronisation, or a plug-in called at a point where its host forbids
// cudaMalloc.  Those callers cannot create a communicator, because a
// communicator allocates its workspace.  This entry point needs none: the
// scratch memory of the kernel (low-latency inbox lines and per-block
// counters) is a fixed array compiled into the library.
//
// The kernel is the library's low-latency one-shot all-reduce
// (ar_oneshot_ll_kernel), launched once for all `nranks` buffers as a
// cooperative grid, exactly as an emulated communicator launches it.
#include <cuda_runtime.h>

#include <string.h>

#include <mutex>

#include "../../include/dgn.h"
#include "dgn_kernels.cuh"

namespace dgn {
int report_error(int code, const char* message);  // dgn_host.cu: sets dgn_last_error_string
}

namespace {

using namespace dgn;

constexpr int kStaticBlocks = 4;            // thread blocks per buffer, at most
constexpr long long kStaticSlot = 8192;     // bytes of lines per (block, source): 256 data vectors
constexpr size_t kStaticHead = 512;         // block counters (4 x 64 B), cleared by every call
constexpr size_t kStaticRankBytes = kStaticHead + 2 * (size_t)kStaticBlocks * DGN_MAX_RANKS * kStaticSlot;
constexpr size_t kStaticStatusOff = (size_t)DGN_MAX_RANKS * kStaticRankBytes;  // error words, never cleared by a call
constexpr size_t kStaticBytes = kStaticStatusOff + 256;  // 4,198,656 bytes
constexpr long long kStaticMaxMessage = (long long)kStaticBlocks * (kStaticSlot / 32) * 16;  // 16 KiB

// The scratch memory.  Every device that loads this library holds one copy
// until the process exits.  In host code this name is only a stand-in for the
// device array; its device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

std::mutex g_setup_mutex;
unsigned char* g_scratch_addr[64] = {};

// Once per device, with that device current: the device address of the array.
int scratch_address(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return report_error(DGN_ERR_CUDA, cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return report_error(DGN_ERR_UNSUPPORTED, "device index beyond 63");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      return report_error(DGN_ERR_CUDA, "cudaGetSymbolAddress failed for the static scratch array");
    }
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[dev];
  return DGN_OK;
}

const void* static_kernel(int dtype) {
  switch (dtype) {
    case DGN_U8: return (const void*)ar_oneshot_ll_kernel<uint8_t, false>;
    case DGN_I8: return (const void*)ar_oneshot_ll_kernel<int8_t, false>;
    case DGN_I32: return (const void*)ar_oneshot_ll_kernel<int32_t, false>;
    case DGN_I64: return (const void*)ar_oneshot_ll_kernel<int64_t, false>;
    case DGN_F16: return (const void*)ar_oneshot_ll_kernel<__half, false>;
    case DGN_BF16: return (const void*)ar_oneshot_ll_kernel<__nv_bfloat16, false>;
    case DGN_F32: return (const void*)ar_oneshot_ll_kernel<float, false>;
    case DGN_F64: return (const void*)ar_oneshot_ll_kernel<double, false>;
    default: return nullptr;
  }
}

}  // namespace

extern "C" int dgn_allreduce_static(int nranks, const void* const* in_ptrs, void* const* out_ptrs,
                                    int64_t count, int dtype, int redop, void* stream) {
  if (nranks < 1 || nranks > DGN_MAX_RANKS)
    return report_error(DGN_ERR_ARG, "dgn_allreduce_static: nranks must be 1..8");
  const size_t es = dgn_dtype_size(dtype);
  if (es == 0) return report_error(DGN_ERR_ARG, "dgn_allreduce_static: unknown dtype");
  if (redop < DGN_SUM || redop > DGN_MAX) return report_error(DGN_ERR_ARG, "dgn_allreduce_static: unknown reduction");
  if (redop == DGN_MEAN && dtype <= DGN_I64)
    return report_error(DGN_ERR_UNSUPPORTED, "MEAN is defined for floating-point types only");
  if (count < 0) return report_error(DGN_ERR_ARG, "dgn_allreduce_static: negative count");
  if (count == 0) return DGN_OK;
  if ((long long)count * (long long)es > kStaticMaxMessage)
    return report_error(DGN_ERR_ARG,
                        "dgn_allreduce_static: message larger than the 16384-byte limit of the static "
                        "scratch array; use a communicator (dgn_allreduce) for larger messages");
  if (!in_ptrs || !out_ptrs) return report_error(DGN_ERR_ARG, "dgn_allreduce_static: null pointer list");
  for (int r = 0; r < nranks; ++r)
    if (!in_ptrs[r] || !out_ptrs[r]) return report_error(DGN_ERR_ARG, "dgn_allreduce_static: null buffer");

  unsigned char* base = nullptr;
  int rc = scratch_address(&base);
  if (rc != DGN_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  const long long nvec = ((long long)count * (long long)es + 15) / 16;
  const long long slot_vecs = kStaticSlot / 32;
  int blocks = (int)((nvec + slot_vecs - 1) / slot_vecs);
  const int cv = (int)((nvec + blocks - 1) / blocks);

  // The array keeps the previous call's lines and counters; with the
  // counters cleared every call uses flag value 1, so the lines this call
  // polls must not hold an old 1.  One memset covers the counters and the
  // parity-0 lines of all `nranks` buffers.
  const size_t used = (size_t)(nranks - 1) * kStaticRankBytes + kStaticHead +
                      (size_t)kStaticBlocks * nranks * kStaticSlot;
  cudaError_t e = cudaMemsetAsync(base, 0, used, s);
  if (e != cudaSuccess) return report_error(DGN_ERR_CUDA, cudaGetErrorString(e));

  OpParams P;
  memset(&P, 0, sizeof(P));
  for (int r = 0; r < nranks; ++r) {
    PeerTable& t = P.peers[r];
    for (int j = 0; j < nranks; ++j) {
      unsigned char* region = base + (size_t)j * kStaticRankBytes;
      t.flags[j] = reinterpret_cast<u64*>(region);  // not used by this kernel
      t.ll[j] = reinterpret_cast<char*>(region + kStaticHead);
    }
    unsigned char* mine = base + (size_t)r * kStaticRankBytes;
    t.blk = reinterpret_cast<BlockState*>(mine);
    // One error word per buffer, behind everything a call clears: a block that
    // gives up leaves DGN_ERR_TIMEOUT there until dgn_allreduce_static_status
    // reads (and, if asked, clears) it.
    t.status = reinterpret_cast<int*>(base + kStaticStatusOff) + r;
    t.rank = r;
    t.nranks = nranks;
    t.max_blocks = kStaticBlocks;
    t.ll_max_blocks = kStaticBlocks;
    t.slot_bytes = 0;
    t.ll_slot_bytes = kStaticSlot;
    P.ra[r].in = in_ptrs[r];
    P.ra[r].out = out_ptrs[r];
    P.ra[r].table = nullptr;
  }
  P.count = count;
  P.nvec = nvec;
  P.wait_ns = 2000000000ull;  // a block gives up after 2 s instead of spinning forever
  P.scale = (double)(1.f / (float)nranks);
  P.ntensors = 1;
  P.rounds = 1;
  P.cv = cv;
  P.redop = redop;
  const void* fn = static_kernel(dtype);
  void* args[1] = {&P};
  // All blocks of all buffers wait on one another's lines, so they must be
  // resident together: a cooperative launch guarantees that.
  e = cudaLaunchCooperativeKernel(fn, dim3(blocks, nranks), dim3(256), args, 0, s);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return report_error(DGN_ERR_CUDA, cudaGetErrorString(e));
  }
  return DGN_OK;
}

// Error word of the static path on the current device: DGN_OK, or
// DGN_ERR_TIMEOUT once a block of an earlier dgn_allreduce_static call gave up
// waiting (its outputs are then incomplete).  Waits for the device's work on
// the legacy default stream's terms (a blocking 32-byte copy); allocates nothing.
extern "C" int dgn_allreduce_static_status(int clear) {
  unsigned char* base = nullptr;
  int rc = scratch_address(&base);
  if (rc != DGN_OK) return rc;
  int words[DGN_MAX_RANKS] = {};
  cudaError_t e = cudaMemcpy(words, base + kStaticStatusOff, sizeof(words), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return report_error(DGN_ERR_CUDA, cudaGetErrorString(e));
  int status = DGN_OK;
  for (int r = 0; r < DGN_MAX_RANKS; ++r)
    if (words[r] != 0) status = words[r];
  if (status != DGN_OK && clear) {
    e = cudaMemset(base + kStaticStatusOff, 0, sizeof(words));
    if (e != cudaSuccess) return report_error(DGN_ERR_CUDA, cudaGetErrorString(e));
  }
  if (status != DGN_OK) report_error(status, "a block of dgn_allreduce_static gave up waiting; outputs of that call are incomplete");
  return status;
}
