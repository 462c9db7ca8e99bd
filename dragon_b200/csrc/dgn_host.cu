// Host side of the dgn C-ABI: communicator bootstrap (symmetric workspace,
// handle exchange, peer mapping), launch planning and the collective entry
// points declared in include/dgn.h.
//
// The reference reaches its collectives through CollectiveOpImpl
// (dragon/operators/distributed/collective_op_impl.h:22-158), which forwards
// to MPI_* or nccl* library calls; here each entry point plans and launches
// its hand-written kernel (dgn_kernels.cuh, dgn_zero.cuh) on the caller's
// stream: one launch per collective, two for the sharded optimizer step.
#include <cuda_runtime.h>

#include <dirent.h>
#include <errno.h>
#include <fcntl.h>
#include <signal.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <mutex>
#include <deque>
#include <string>
#include <vector>

#include "../../include/dgn.h"
#include "dgn_kernels.cuh"
#include "dgn_nvls.h"
#include "dgn_update.cuh"
#include "dgn_zero.cuh"

namespace dgn {
// Defined in the per-dtype instantiation units.
const void* reduce_kernel_fn_0(int, bool);
const void* reduce_kernel_fn_1(int, bool);
const void* reduce_kernel_fn_2(int, bool);
const void* reduce_kernel_fn_3(int, bool);
const void* reduce_kernel_fn_4(int, bool);
const void* reduce_kernel_fn_5(int, bool);
const void* reduce_kernel_fn_6(int, bool);
const void* reduce_kernel_fn_7(int, bool);
const void* allgather_kernel_fn();
const void* allgather_pull_kernel_fn();
const void* allgather_ll_kernel_fn();
const void* broadcast_kernel_fn();
const void* broadcast_scatter_kernel_fn();
const void* gather_flow_kernel_fn(bool through_switch);
const void* local_copy_kernel_fn(int es, bool table);
const void* zero_kernel_fn(int dtype, int which);  // dgn_zero_inst.cu
const void* update_kernel_fn(int kind);             // dgn_update_inst.cu
}  // namespace dgn

using namespace dgn;

namespace {

thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define DGN_CUDA(expr)                                                              \
  do {                                                                              \
    cudaError_t e__ = (expr);                                                       \
    if (e__ != cudaSuccess)                                                         \
      return fail(DGN_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                  __FILE__, __LINE__);                                              \
  } while (0)

const size_t kElemSize[8] = {1, 1, 4, 8, 2, 2, 4, 8};

long long env_ll(const char* name, long long dflt) {
  const char* s = getenv(name);
  if (!s || !*s) return dflt;
  char* end = nullptr;
  long long v = strtoll(s, &end, 10);
  return (end && *end == '\0') ? v : dflt;
}

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

constexpr uint32_t kMagic = 0x44474e31u;  // "DGN1"

struct Handle {  // what one rank tells the others; padded to DGN_HANDLE_BYTES
  uint32_t magic, version;
  int32_t pid, device, rank, nranks, max_blocks, pad;
  int64_t slot_bytes;
  uint64_t total_bytes;
  uint64_t base_ptr;
  uint64_t host_id;
  cudaIpcMemHandle_t ipc;
  int32_t nvls_capable;
  char nvls_sock[64];  // rank 0: name of the multicast rendezvous socket
  uint64_t symm_bytes;  // symmetric arena; must agree on all ranks
  uint64_t session;     // drawn when the communicator is created: tells this run's rendezvous files from stale ones
};
static_assert(sizeof(Handle) <= DGN_HANDLE_BYTES, "handle too large");

uint64_t host_identity() {
  uint64_t h = 1469598103934665603ull;
  auto mix = [&](const char* s) {
    for (; *s; ++s) h = (h ^ (unsigned char)*s) * 1099511628211ull;
  };
  char buf[256] = "";
  gethostname(buf, sizeof(buf) - 1);
  mix(buf);
  FILE* f = fopen("/proc/sys/kernel/random/boot_id", "r");
  if (f) {
    if (fgets(buf, sizeof(buf), f)) mix(buf);
    fclose(f);
  }
  return h;
}

struct Geometry {
  int nranks = 1, max_blocks = 0, ll_max_blocks = 0;
  long long slot_bytes = 0, ll_slot_bytes = 0;
  size_t flags_bytes = 0, blk_off = 0, flow_state_off = 0, flow_flags_off = 0, stage_off = 0, ll_off = 0,
         ll2_off = 0, ring_off = 0, ring_bytes = 0, total = 0;
};

// Workspace layout: [flags][block states][flow state][flow flags] | [staging] |
// [low-latency region] | [two-shot low-latency region] | [ring of the staged
// dataflow all-reduce without the switch].
Geometry make_geometry(int nranks) {
  Geometry g;
  g.nranks = nranks;
  g.max_blocks = (int)env_ll("DGN_MAX_BLOCKS", 160);
  if (g.max_blocks < 1) g.max_blocks = 1;
  if (g.max_blocks > 1024) g.max_blocks = 1024;
  g.slot_bytes = env_ll("DGN_SLOT_BYTES", 128 * 1024);
  if (g.slot_bytes < 4096) g.slot_bytes = 4096;
  g.slot_bytes = (g.slot_bytes + 4095) & ~4095ll;
  g.ll_max_blocks = (int)env_ll("DGN_LL_MAX_BLOCKS", 64);
  if (g.ll_max_blocks < 1) g.ll_max_blocks = 1;
  if (g.ll_max_blocks > g.max_blocks) g.ll_max_blocks = g.max_blocks;
  g.ll_slot_bytes = env_ll("DGN_LL_SLOT_BYTES", 64 * 1024);
  if (g.ll_slot_bytes < 4096) g.ll_slot_bytes = 4096;
  g.ll_slot_bytes = (g.ll_slot_bytes + 4095) & ~4095ll;
  g.flags_bytes = (size_t)g.max_blocks * kChannels * kMaxRanks * sizeof(u64);
  g.blk_off = g.flags_bytes;
  size_t head = g.blk_off + (size_t)g.max_blocks * sizeof(BlockState);
  g.flow_state_off = (head + 255) & ~(size_t)255;
  // Two states (staged all-reduce, staged gather) and four kinds of flag words.
  g.flow_flags_off = g.flow_state_off + ((2 * sizeof(FlowState) + 255) & ~(size_t)255);
  head = g.flow_flags_off + 4 * (size_t)kFlowSlots * kMaxRanks * sizeof(u64);
  g.stage_off = (head + 4095) & ~(size_t)4095;
  g.ll_off = g.stage_off + 2 * (size_t)g.max_blocks * 2 * (size_t)(2 * nranks) * (size_t)g.slot_bytes;
  g.ll2_off = g.ll_off + 2 * (size_t)g.ll_max_blocks * (size_t)nranks * (size_t)g.ll_slot_bytes;
  g.ring_off = g.ll2_off + 2 * (size_t)g.ll_max_blocks * 2 * (size_t)nranks * (size_t)g.ll_slot_bytes;
  // The multicast version keeps its ring in the multicast-bound buffer; this
  // one serves communicators without the switch (and virtual ranks).
  long long ring = nranks > 1 ? env_ll("DGN_RING_BYTES", 64ll << 20) : 0;
  if (ring < 0) ring = 0;
  g.ring_bytes = ((size_t)ring + 4095) & ~(size_t)4095;
  g.total = g.ring_off + g.ring_bytes;
  return g;
}

struct TableEntry {
  std::vector<const void*> in;
  std::vector<void*> out;
  std::vector<int64_t> counts;
  int es = 0;
  TensorEnt* d_table = nullptr;
  TensorEnt* h_table = nullptr;  // pinned
  int nt = 0;                    // non-empty tensors
  long long nvec = 0;
  uint64_t last_use = 0;
  cudaStream_t upload_stream = nullptr;  // the table was copied to the device on this stream ...
  cudaEvent_t uploaded = nullptr;        // ... and this event follows the copy
};

struct Plan {
  int variant = 0, blocks = 1, threads = 512, cv = 1, rounds = 1;
  int unroll = 8;  // multicast kernels: loads in flight per thread
  // staged dataflow all-reduce: reducing / copy-in blocks (the rest copy out), ring slots
  int flow_nsw = 0, flow_nin = 0, flow_depth = 0;
  // staged gather: mode bits and the inbox of the scattering broadcast (bytes from the workspace base)
  int flow_mode = 0;
  long long inbox_off = 0;
};

enum OpKind { kOpAllReduce = 0, kOpReduceScatter, kOpAllGather, kOpBroadcast, kOpZeroReduce, kOpZeroUpdate,
              kOpAllReduceUpdate };

inline bool is_zero_kind(int kind) { return kind == kOpZeroReduce || kind == kOpZeroUpdate; }

// Hyper-parameters of one sharded optimizer step; identical on every rank.
struct ZeroHyper {
  float lr = 0, beta1 = 0, beta2 = 0, eps = 0, wd = 0, grad_scale = 1, clip_norm = 0, clip_value = 0;
  int check_finite = 0, use_lr_scales = 0;
};

// Hyper-parameters of the all-reduce fused with the optimizer update; identical on every rank.
struct UpdHyper {
  int kind = 0;
  float lr = 0, a = 0, b = 0, eps = 0, wd = 0, grad_scale = 1, clip_value = 0;
};

struct OpDesc {
  int kind = 0, dtype = 0, redop = 0, root = 0, ntensors = 1;
  long long count = 0;  // elements (AR single / RS per-rank block / bucket of a sharded step) or bytes (AG / BC)
  long long nvec = 0;
  const void* in = nullptr;
  void* out = nullptr;
  const TensorEnt* table = nullptr;
  cudaStream_t stream = nullptr;
  ZeroRank zr = {};  // sharded optimizer step only
  ZeroHyper zh;
  const UpdEnt* utable = nullptr;  // all-reduce fused with the optimizer update only
  UpdHyper uh;
};

// Device table of a sharded optimizer step, cached on the tensor list.
struct ZeroTableEntry {
  std::vector<const void*> grads;
  std::vector<void*> params;
  std::vector<int64_t> counts;
  std::vector<float> lrs;
  int es = 0;
  ZeroEnt* d_table = nullptr;
  ZeroEnt* h_table = nullptr;  // pinned
  int nt = 0;                  // non-empty tensors
  long long total = 0;
  uint64_t last_use = 0;
  cudaStream_t upload_stream = nullptr;
  cudaEvent_t uploaded = nullptr;
};

// Device table of an all-reduce fused with the optimizer update, cached on the tensor list.
struct UpdTableEntry {
  std::vector<const void*> grads;
  std::vector<void*> params, m, v;
  std::vector<int64_t> counts;
  UpdEnt* d_table = nullptr;
  UpdEnt* h_table = nullptr;  // pinned
  int nt = 0;
  long long nvec = 0;
  uint64_t last_use = 0;
  cudaStream_t upload_stream = nullptr;
  cudaEvent_t uploaded = nullptr;
};

struct Team;

}  // namespace

struct dgn_comm {
  int rank = 0, nranks = 1, device = 0, num_sms = 148;
  Geometry geo;
  void* base = nullptr;  // workspace
  int* status_host = nullptr;
  int* status_dev = nullptr;
  void* peer_base[kMaxRanks] = {};
  bool peer_ipc[kMaxRanks] = {};
  PeerTable table;  // this rank's view of the team, copied into every launch
  bool connected = false;
  u64 wait_ns = 5000000000ull;
  int tune_variant = 0, tune_blocks = 0, tune_threads = 0;
  long long tune_chunk = 0;
  long long oneshot_max_bytes = -1, ll_max_bytes = -1, ll2_max_bytes = -1;
  long long bcast_scatter_min_bytes = 1ll << 20;
  long long allgather_pull_min_bytes = 1ll << 62;  // per-rank block from which peers pull instead of being pushed to
  long long ll_allgather_max_bytes = 512ll << 10;  // per-rank block of the low-latency all-gather (set per rank count)
  bool fused_twoshot = false;  // DGN_TWOSHOT_FUSED=1: lock-step two-shot kernel instead of the warp-specialised one
  Team* team = nullptr;
  std::vector<TableEntry> tables;
  std::vector<ZeroTableEntry> zero_tables;
  std::vector<UpdTableEntry> upd_tables;
  uint64_t table_clock = 0;
  Plan last_plan;
  std::string rdv_ok_file;
  // host-memory all-reduce: its own stream and two 4 KiB staging buffers
  cudaStream_t host_stream = nullptr;
  void* host_dev = nullptr;
  void* host_pin = nullptr;
  uint64_t session = 0;                // pid and creation time; goes into the handle
  cudaStream_t last_stream = nullptr;  // stream of the latest collective
  bool has_last_stream = false;
  // NVSwitch multicast staging (optional)
  NvlsBuffer* nvls = nullptr;
  bool nvls_capable = false;
  char nvls_sock[64] = {};
  long long nvls_min_bytes = 0;
  // Staged gather (gather_flow_kernel): ring at the start of the multicast-bound
  // buffer, chunk size per source, pushing blocks (0: automatic), thresholds.
  size_t gather_ring_bytes = 0;
  long long gather_chunk_bytes = 0, nvls_allgather_min_bytes = 0, allgather_ring_min_bytes = 0;
  long long bcast_shard_min_bytes = 0;  // smallest staged broadcast whose root scatters shards
  int gather_push_blocks = 0, gather_forward_blocks = 0, gather_mode = 0;
  size_t nvls_bytes = 0;
  // Symmetric arena: the tail of the multicast-bound buffer, handed out by
  // dgn_comm_symm_alloc; buffers in it can be reduced in place by the switch.
  size_t symm_bytes = 0, symm_off = 0, symm_used = 0;
  long long symm_min_bytes = 0;
  // Staged dataflow all-reduce (ar_flow_kernel): ring inside the multicast-bound
  // buffer, chunk size, block split, ring slots, loads in flight (0: automatic).
  size_t flow_ring_off = 0, flow_ring_bytes = 0;
  long long flow_chunk_bytes = 0;
  int flow_switch_blocks = 0, flow_in_blocks = 0, flow_out_blocks = 0, flow_depth = 0, unroll = 0, pattern = 0;
  long long nvls_bcast_min_bytes = 0;  // smallest broadcast that goes through the switch
  bool plan_query = false, plan_query_in_symm = false;  // dgn_plan_query: no device, no real buffers
};

namespace {

struct Team {
  int n = 0, device = 0;
  std::vector<dgn_comm*> members;
  std::deque<OpDesc> pending[kMaxRanks];
  int alive = 0;
};

const void* reduce_fn(int dtype, int kind, bool table);

// Loads every kernel of the library on the current device.  With lazy module
// loading the first launch of a kernel has to load its module, which can wait
// for the device to go idle; a device that is already spinning in a
// collective, waiting for this very launch on a peer, would never go idle.
// Touching each kernel once, before any collective, takes loading out of the
// launch path.
int preload_kernels() {
  cudaFuncAttributes attr;
  for (int dtype = 0; dtype < 8; ++dtype) {
    for (int kind = 0; kind <= 8; ++kind) {
      for (int table = 0; table < 2; ++table) {
        const void* fn = reduce_fn(dtype, kind, table != 0);
        if (fn) DGN_CUDA(cudaFuncGetAttributes(&attr, fn));
      }
    }
  }
  DGN_CUDA(cudaFuncGetAttributes(&attr, allgather_kernel_fn()));
  DGN_CUDA(cudaFuncGetAttributes(&attr, allgather_pull_kernel_fn()));
  DGN_CUDA(cudaFuncGetAttributes(&attr, allgather_ll_kernel_fn()));
  DGN_CUDA(cudaFuncGetAttributes(&attr, broadcast_kernel_fn()));
  DGN_CUDA(cudaFuncGetAttributes(&attr, broadcast_scatter_kernel_fn()));
  DGN_CUDA(cudaFuncGetAttributes(&attr, gather_flow_kernel_fn(true)));
  DGN_CUDA(cudaFuncGetAttributes(&attr, gather_flow_kernel_fn(false)));
  const int sizes[4] = {1, 2, 4, 8};
  for (int es : sizes)
    for (int table = 0; table < 2; ++table)
      DGN_CUDA(cudaFuncGetAttributes(&attr, local_copy_kernel_fn(es, table != 0)));
  const int zero_types[3] = {DGN_F16, DGN_BF16, DGN_F32};
  for (int dtype : zero_types)
    for (int which = 0; which < 3; ++which)
      DGN_CUDA(cudaFuncGetAttributes(&attr, zero_kernel_fn(dtype, which)));
  for (int kind = 0; kind < 4; ++kind) DGN_CUDA(cudaFuncGetAttributes(&attr, update_kernel_fn(kind)));
  return DGN_OK;
}

thread_local bool g_skip_nvls = false;  // set while emulated ranks are created
thread_local long long g_symm_request = -1;  // dgn_comm_init_symmetric: arena bytes for the next init_local
std::mutex g_registry_mutex;
std::map<uint64_t, dgn_comm*>& registry() {  // workspace base -> communicator, this process
  static std::map<uint64_t, dgn_comm*> r;
  return r;
}

int alloc_workspace(dgn_comm* c) {
  DeviceGuard g(c->device);
  int rc = preload_kernels();
  if (rc != DGN_OK) return rc;
  DGN_CUDA(cudaMalloc(&c->base, c->geo.total));
  DGN_CUDA(cudaMemset(c->base, 0, c->geo.stage_off));
  DGN_CUDA(cudaMemset(static_cast<char*>(c->base) + c->geo.ll_off, 0, c->geo.total - c->geo.ll_off));
  DGN_CUDA(cudaHostAlloc((void**)&c->status_host, 64, cudaHostAllocMapped | cudaHostAllocPortable));
  *c->status_host = 0;
  DGN_CUDA(cudaHostGetDevicePointer((void**)&c->status_dev, c->status_host, 0));
  DGN_CUDA(cudaStreamCreateWithFlags(&c->host_stream, cudaStreamNonBlocking));
  DGN_CUDA(cudaMalloc(&c->host_dev, 4096));
  DGN_CUDA(cudaHostAlloc(&c->host_pin, 4096, cudaHostAllocDefault));
  DGN_CUDA(cudaDeviceSynchronize());
  cudaDeviceProp prop;
  DGN_CUDA(cudaGetDeviceProperties(&prop, c->device));
  c->num_sms = prop.multiProcessorCount;
  return DGN_OK;
}

void fill_peer_table(const dgn_comm* c, PeerTable* t) {
  memset(t, 0, sizeof(*t));
  for (int j = 0; j < c->nranks; ++j) {
    char* b = static_cast<char*>(c->peer_base[j]);
    t->flags[j] = reinterpret_cast<u64*>(b);
    t->stage[j] = b + c->geo.stage_off;
    t->ll[j] = b + c->geo.ll_off;
    t->ll2[j] = b + c->geo.ll2_off;
  }
  t->blk = reinterpret_cast<BlockState*>(static_cast<char*>(c->base) + c->geo.blk_off);
  t->status = c->status_dev;
  t->rank = c->rank;
  t->nranks = c->nranks;
  t->max_blocks = c->geo.max_blocks;
  t->ll_max_blocks = c->geo.ll_max_blocks;
  t->slot_bytes = c->geo.slot_bytes;
  t->ll_slot_bytes = c->geo.ll_slot_bytes;
  t->nvls_uc = t->nvls_mc = nullptr;
  if (c->nvls) nvls_pointers(c->nvls, &t->nvls_uc, &t->nvls_mc);
  t->ring_gather_off = (long long)(c->geo.ring_off + c->geo.ring_bytes / 2);
  t->flow_state_off = (long long)c->geo.flow_state_off;
  t->flow_flags_off = (long long)c->geo.flow_flags_off;
  t->ring_off = (long long)c->geo.ring_off;
  t->nvls_ring_off = (long long)c->flow_ring_off;
}

const void* reduce_fn(int dtype, int kind, bool table) {
  switch (dtype) {
    case DGN_U8: return reduce_kernel_fn_0(kind, table);
    case DGN_I8: return reduce_kernel_fn_1(kind, table);
    case DGN_I32: return reduce_kernel_fn_2(kind, table);
    case DGN_I64: return reduce_kernel_fn_3(kind, table);
    case DGN_F16: return reduce_kernel_fn_4(kind, table);
    case DGN_BF16: return reduce_kernel_fn_5(kind, table);
    case DGN_F32: return reduce_kernel_fn_6(kind, table);
    case DGN_F64: return reduce_kernel_fn_7(kind, table);
    default: return nullptr;
  }
}

long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

long long default_ll_max(int n) {
  // Flag-in-data lines carry 8 bytes of data per 16 sent and every rank sends
  // its whole message to every peer: (n - 1) * 2 * S bytes per rank.
  // Measured: n = 2 up to 2 MiB, the most the line region holds (24.2 / 27.4 us
  // at 1.5 / 2 MiB against 31.0 / 31.7 us for two-shot); n = 4 up to 512 KiB.
  if (n <= 2) return 2ll << 20;
  if (n <= 4) return 512ll << 10;
  return 128ll << 10;
}

long long default_ll2_max(int n) {
  // Two ranks gain nothing from sharding (one-shot moves the same bytes).
  // Measured at n = 8 (replayed graphs): best from 256 KiB to 2 MiB.
  if (n <= 2) return 0;
  return 2ll << 20;
}

long long default_oneshot_max(int n) {
  // Above these sizes the (n - 1)x link traffic of one-shot costs more than
  // the second flag exchange of two-shot.
  if (n <= 2) return 1ll << 20;
  if (n <= 4) return 1ll << 20;
  return 256ll << 10;
}

// True if the all-reduce can run in place in the symmetric arena: one tensor,
// in == out, inside the arena, a whole number of 16-byte vectors (the switch
// reduces whole vectors, so a ragged tail would touch its neighbour's bytes).
bool symm_inplace_ok(const dgn_comm* c, const OpDesc& d) {
  if (!c->nvls || c->symm_bytes == 0 || d.ntensors != 1 || d.in != d.out || !d.in) return false;
  if (c->plan_query)
    return c->plan_query_in_symm && ((d.count * (long long)kElemSize[d.dtype]) & 15) == 0;
  char *uc = nullptr, *mc = nullptr;
  nvls_pointers(c->nvls, &uc, &mc);
  const char* lo = uc + c->symm_off;
  const char* p = static_cast<const char*>(d.in);
  const long long bytes = d.count * (long long)kElemSize[d.dtype];
  if (p < lo || p + bytes > lo + c->symm_bytes) return false;
  return ((uintptr_t)p & 15u) == 0 && (bytes & 15) == 0;
}

// Launch shape of the staged dataflow all-reduce (ar_flow_kernel) over a ring of
// `ring_bytes`; false if the ring or the grid is too small for it.
bool plan_flow(const dgn_comm* c, const OpDesc& d, int block_cap, long long ring_bytes, int variant, Plan* out) {
  const int n = c->nranks;
  const long long bytes = d.nvec * 16;
  int total = c->num_sms;  // one block per SM, all resident (the blocks wait for one another)
  if (total > c->geo.max_blocks) total = c->geo.max_blocks;
  if (block_cap > 0 && block_cap < total) total = block_cap;
  if (total < 3 || ring_bytes < 2 * 4096) return false;
  // Chunks: half of the message, between 1 and 16 MiB.  Measured at 8 ranks (8
  // reducing blocks): 16 MiB chunks are best from 32 MiB to 1 GiB (115 / 189 /
  // 330 / 611 / 2311 us at 32 / 64 / 128 / 256 / 1024 MiB); two chunks are best
  // at 8 and 16 MiB (56 and 77 us, against 64 and 89 us with four); smaller
  // chunks pay a few microseconds each for their flags, larger ones fill and
  // drain longer.
  long long chunk = c->flow_chunk_bytes;
  if (c->tune_chunk >= 4096) chunk = c->tune_chunk;
  if (chunk <= 0) {
    chunk = ceil_div(bytes, 2);
    if (chunk < (1ll << 20)) chunk = 1ll << 20;
    if (chunk > (16ll << 20)) chunk = 16ll << 20;
  }
  if (chunk > ring_bytes / 2) chunk = ring_bytes / 2;
  long long cv = ceil_div(chunk, 16 * (long long)n) * n;  // whole vectors, equal shards
  if (cv * 16 > ring_bytes / 2) cv = (ring_bytes / 2) / (16 * (long long)n) * n;
  if (cv < n || cv > 0x7fffffff) return false;
  const long long K = ceil_div(d.nvec, cv);
  if (K > 0x7fffffff) return false;
  long long depth = ring_bytes / (cv * 16);
  if (depth > kFlowSlots) depth = kFlowSlots;
  if (c->flow_depth > 0 && c->flow_depth < depth) depth = c->flow_depth;
  if (depth > K) depth = K;
  if (depth < 1) depth = 1;
  // Few reducing blocks: the switch path saturates with about a quarter of a
  // megabyte of loads in flight per rank, and every reducing block adds a fence
  // per chunk.  Measured at 8 ranks, 256 MiB, 16 MiB chunks: 8 blocks 615 us,
  // 16 blocks 690 us, 32 blocks 797 us.
  int nsw = c->flow_switch_blocks > 0 ? c->flow_switch_blocks : (total >= 64 ? 8 : (total + 6) / 7);
  if (c->tune_blocks > 0) nsw = c->tune_blocks;
  if (nsw > total - 2) nsw = total - 2;
  if (nsw < 1) nsw = 1;
  int nin = c->flow_in_blocks > 0 ? c->flow_in_blocks : (total - nsw) / 2;
  if (nin > total - nsw - 1) nin = total - nsw - 1;
  if (nin < 1) nin = 1;
  int nout = c->flow_out_blocks > 0 ? c->flow_out_blocks : total - nsw - nin;
  if (nout > total - nsw - nin) nout = total - nsw - nin;
  if (nout < 1) return false;
  Plan p;
  p.variant = variant;
  p.threads = c->tune_threads > 0 ? c->tune_threads : 512;
  if (p.threads > kMaxThreads) p.threads = kMaxThreads;
  p.threads = p.threads / 32 * 32;
  if (p.threads < 64) p.threads = 64;  // a reducing block needs a data warp and its signal warp
  p.blocks = nsw + nin + nout;
  p.cv = (int)cv;
  p.rounds = (int)K;
  p.unroll = c->unroll > 0 ? c->unroll : 4;
  p.flow_nsw = nsw;
  p.flow_nin = nin;
  p.flow_depth = (int)depth;
  *out = p;
  return true;
}

// Launch shape of the staged gather (gather_flow_kernel: all-gather and
// broadcast); false if ring, inbox or grid are too small.  Variant NVLS keeps the
// ring in the multicast-bound buffer and the inbox of the scattering broadcast
// in the gather half of the workspace ring; RING / RING_PULL keep both in that
// half (ring first, inbox behind it).
bool plan_gather(const dgn_comm* c, const OpDesc& d, int block_cap, int variant, Plan* out) {
  const int n = c->nranks;
  const bool gather = d.kind == kOpAllGather;
  const bool pull = variant == DGN_VARIANT_RING_PULL;
  if (pull && !gather) return false;
  const long long bytes = d.nvec * 16;  // per block (all-gather) / of the message (broadcast)
  // Broadcast: from three ranks on the root scatters shards and every rank
  // multicasts its own (no rank has to feed the switch alone).
  bool scatter = !gather && n >= 5 && bytes >= c->bcast_shard_min_bytes;  // 4 ranks: 303 us scattered, 181 us alone at 64 MiB
  if (c->gather_mode == 1) scatter = false;
  if (c->gather_mode == 2 && !gather && n >= 2) scatter = true;
  const long long half = (long long)c->geo.ring_bytes / 2;
  if (scatter && half < 2 * 4096) scatter = false;  // no room for the inboxes: the root multicasts alone
  const int nsrc = (gather || scatter) ? n : 1;
  const int nreg = pull ? 1 : nsrc;
  const long long ring_bytes = variant == DGN_VARIANT_NVLS ? (long long)c->gather_ring_bytes : half;
  int total = c->num_sms;
  if (total > c->geo.max_blocks) total = c->geo.max_blocks;
  if (block_cap > 0 && block_cap < total) total = block_cap;
  if (total < 2 || ring_bytes < 2ll * (nreg + 1) * 4096) return false;
  // Chunk sizes from the sweeps at 8 ranks.  All-gather through the switch: half
  // a block up to 2 MiB (78 us at 4 MiB blocks, 835 us at 64 MiB); pulling: a
  // quarter up to 4 MiB.  Broadcast with the root alone: half the message up to
  // 8 MiB (34 / 66 / 196 us at 4 / 16 / 64 MiB); scattered: an eighth, 1 to 8 MiB
  // (181 us at 64 MiB with 8 MiB chunks, 212 us with 4 MiB, 192 us with 16 MiB).
  long long chunk = c->gather_chunk_bytes;
  if (c->tune_chunk >= 4096) chunk = c->tune_chunk;
  if (chunk <= 0) {
    long long lo = 256ll << 10, hi = 8ll << 20;
    if (gather) {
      chunk = ceil_div(bytes, pull ? 4 : 2);
      hi = pull ? (4ll << 20) : (2ll << 20);
    } else if (scatter) {
      chunk = ceil_div(bytes, 8);
      lo = 1ll << 20;
    } else {
      chunk = ceil_div(bytes, 2);
    }
    if (chunk < lo) chunk = lo;
    if (chunk > hi) chunk = hi;
  }
  long long cv = ceil_div(chunk, 16 * (long long)(gather ? 1 : nsrc));  // per source
  // At least two slots of ring (and of inbox, where the two share the half).
  const bool shared = variant != DGN_VARIANT_NVLS;
  long long cv_max = ring_bytes / (2ll * (nreg + (shared && scatter ? 1 : 0)) * 16);
  if (scatter && !shared && cv_max > half / (2 * 16)) cv_max = half / (2 * 16);
  if (cv > cv_max) cv = cv_max;
  const long long per_src = gather ? d.nvec : ceil_div(d.nvec, nsrc);
  if (cv > per_src) cv = per_src;
  if (cv < 1 || cv > 0x7fffffff) return false;
  const long long K = ceil_div(d.nvec, gather ? cv : cv * nsrc);
  if (K > 0x7fffffff) return false;
  long long depth = ring_bytes / ((nreg + (shared && scatter ? 1 : 0)) * cv * 16);
  if (scatter && !shared && depth > half / (cv * 16)) depth = half / (cv * 16);
  if (depth > kFlowSlots) depth = kFlowSlots;
  if (c->flow_depth > 0 && c->flow_depth < depth) depth = c->flow_depth;
  if (depth > K) depth = K;
  if (depth < 1) depth = 1;
  Plan p;
  p.variant = variant;
  p.threads = c->tune_threads > 0 ? c->tune_threads : 512;
  if (p.threads > kMaxThreads) p.threads = kMaxThreads;
  p.threads = p.threads / 32 * 32;
  if (p.threads < 64) p.threads = 64;  // a pushing block needs a data warp and its signal warp
  // Pushing blocks.  All-gather: a source sends S while (n - 1) S arrive, and
  // few pushing blocks congest the switch least (2 blocks: 835 us, 8 blocks: 930
  // us at 8 ranks and 64 MiB); when pulling they only copy into the own ring (32
  // blocks: 898 us, 8 blocks: 1128 us).  Broadcast: the root feeds everybody (16
  // blocks alone, 32 when it scatters: 181 us against 197 / 214 us with 16 / 64).
  int npush = c->gather_push_blocks > 0 ? c->gather_push_blocks : gather ? (pull ? 32 : 2) : (scatter ? 32 : 16);
  if (c->tune_blocks > 0) npush = c->tune_blocks;
  const long long per_push = (long long)(p.threads - 32) * 4;  // vectors one block pushes per pass
  const long long root_cv = scatter ? cv * nsrc : cv;
  if (npush > ceil_div(root_cv, per_push)) npush = (int)ceil_div(root_cv, per_push);
  if (npush > total / 2) npush = total / 2;  // small grids (virtual ranks): leave half the blocks to the copies
  if (npush < 1) npush = 1;
  int nfwd = 0;
  if (scatter) {
    nfwd = c->gather_forward_blocks > 0 ? c->gather_forward_blocks : 2;
    if (nfwd > ceil_div(cv, per_push)) nfwd = (int)ceil_div(cv, per_push);
    if (nfwd > total / 2) nfwd = total / 2;
    if (nfwd < 1) nfwd = 1;
  }
  // Copying blocks: enough for the parts of a chunk, no more than the SMs left.
  const int most = npush > nfwd ? npush : nfwd;
  long long nout = ceil_div((long long)nsrc * cv, (long long)p.threads * 4);
  if (nout > total - most) nout = total - most;
  if (nout < 1) nout = 1;
  p.blocks = most + (int)nout;
  p.cv = (int)cv;
  p.rounds = (int)K;
  p.unroll = c->unroll > 0 ? (c->unroll > 8 ? 8 : c->unroll) : (gather ? 8 : 4);
  p.flow_nsw = npush;
  p.flow_nin = nfwd;
  p.flow_depth = (int)depth;
  p.flow_mode = (scatter ? kGatherScatter : 0) | (pull ? kGatherPull : 0);
  p.inbox_off = (long long)c->geo.ring_off + half + (shared ? depth * nreg * cv * 16 : 0);
  *out = p;
  return true;
}

// Chooses variant and launch shape.  `block_cap` bounds the grid (cooperative
// launches must be fully resident).
Plan make_plan(const dgn_comm* c, const OpDesc& d, int block_cap) {
  Plan p;
  const int n = c->nranks;
  const long long slot_vecs = c->geo.slot_bytes / 16;
  int bmax = c->geo.max_blocks;
  if (block_cap > 0 && block_cap < bmax) bmax = block_cap;
  if (c->tune_blocks > 0 && c->tune_blocks < bmax) bmax = c->tune_blocks;
  if (bmax < 1) bmax = 1;
  p.threads = c->tune_threads > 0 ? c->tune_threads : 512;
  if (p.threads > kMaxThreads) p.threads = kMaxThreads;
  if (p.threads < 32) p.threads = 32;
  p.threads = (p.threads / 32) * 32;
  long long cv_cap = slot_vecs;
  if (c->tune_chunk >= 16 && c->tune_chunk / 16 < cv_cap) cv_cap = c->tune_chunk / 16;

  if (d.kind == kOpAllReduce && c->nvls && !c->team &&
      (d.dtype == DGN_F32 || d.dtype == DGN_F16 || d.dtype == DGN_BF16) &&
      (d.redop == DGN_SUM || d.redop == DGN_MEAN)) {
    // NVSwitch multicast: in-switch reduction, about half the link traffic.
    const long long bytes = d.nvec * 16;
    if (symm_inplace_ok(c, d)) {
      bool symm = bytes >= c->symm_min_bytes && c->tune_variant == DGN_VARIANT_AUTO;
      if (c->tune_variant == DGN_VARIANT_SYMM) symm = true;
      if (symm) {
        // No staging: the grid only has to keep enough multimem loads in flight,
        // and the switch path saturates early.  Measured at 8 ranks (64 / 256 MiB):
        // 8 to 32 blocks x 128 or 256 threads with 8 loads per thread all give 163 /
        // 576 us; 64 blocks x 512 threads 206 / 640 us, 148 x 512 up to 660 us.
        if (c->tune_threads <= 0) p.threads = 256;
        const long long vs = ceil_div(d.nvec, n);
        long long b = ceil_div(vs, p.threads);
        int nb = 16;
        if (c->tune_blocks > 0) nb = c->tune_blocks < c->geo.max_blocks ? c->tune_blocks : c->geo.max_blocks;
        if (block_cap > 0 && nb > block_cap) nb = block_cap;
        if (b > nb) b = nb;
        if (b < 1) b = 1;
        p.variant = DGN_VARIANT_SYMM;
        p.blocks = (int)b;
        p.cv = (int)(ceil_div(vs, b) > 0x7fffffff ? 0x7fffffff : ceil_div(vs, b));
        p.rounds = 1;
        p.unroll = c->unroll > 0 ? c->unroll : 8;
        return p;
      }
    }
    bool nvls = bytes >= c->nvls_min_bytes && c->tune_variant == DGN_VARIANT_AUTO;
    if (c->tune_variant == DGN_VARIANT_NVLS) nvls = true;
    if (nvls && plan_flow(c, d, block_cap, (long long)c->flow_ring_bytes, DGN_VARIANT_NVLS, &p)) return p;
  }
  if (d.kind == kOpAllReduce && c->tune_variant == DGN_VARIANT_RING &&
      plan_flow(c, d, block_cap, (long long)c->geo.ring_bytes / 2, DGN_VARIANT_RING, &p))
    return p;
  if (d.kind == kOpAllReduce) {
    const long long bytes = d.nvec * 16;
    // Low-latency one-shot: flag-in-data lines, no barrier at all.
    const long long ll_vecs = c->geo.ll_slot_bytes / 32;  // data vectors per LL slot
    int ll_bmax = c->geo.ll_max_blocks;
    if (block_cap > 0 && block_cap < ll_bmax) ll_bmax = block_cap;
    const bool ll_fits = ceil_div(d.nvec, ll_bmax) <= ll_vecs;
    const long long ll_thr = c->ll_max_bytes >= 0 ? c->ll_max_bytes : default_ll_max(n);
    bool ll = ll_fits && bytes <= ll_thr;
    if (c->tune_variant == DGN_VARIANT_LL) ll = ll_fits;
    else if (c->tune_variant != DGN_VARIANT_AUTO) ll = false;
    if (ll) {
      p.variant = DGN_VARIANT_LL;
      long long b = ceil_div(d.nvec, 256);
      if (c->tune_blocks > 0) b = c->tune_blocks;
      if (b > ll_bmax) b = ll_bmax;
      if (b < 1) b = 1;
      if (ceil_div(d.nvec, b) > ll_vecs) b = ceil_div(d.nvec, ll_vecs);
      p.blocks = (int)b;
      p.cv = (int)ceil_div(d.nvec, b);
      p.rounds = 1;
      if (c->tune_threads <= 0) {
        long long t = ((long long)p.cv + 31) / 32 * 32;
        p.threads = (int)(t < 64 ? 64 : (t > 512 ? 512 : t));
      }
      return p;
    }
    // Low-latency two-shot: shard slices as flag-in-data lines.
    {
      const long long vs = ceil_div(d.nvec, n);
      const bool ll2_fits = ceil_div(vs, ll_bmax) <= ll_vecs;
      const long long ll2_thr = c->ll2_max_bytes >= 0 ? c->ll2_max_bytes : default_ll2_max(n);
      bool ll2 = ll2_fits && bytes <= ll2_thr;
      if (c->tune_variant == DGN_VARIANT_LL2) ll2 = ll2_fits;
      else if (c->tune_variant != DGN_VARIANT_AUTO) ll2 = false;
      if (ll2) {
        p.variant = DGN_VARIANT_LL2;
        long long b = ceil_div(vs, 256);
        if (c->tune_blocks > 0) b = c->tune_blocks;
        if (b > ll_bmax) b = ll_bmax;
        if (b < 1) b = 1;
        if (ceil_div(vs, b) > ll_vecs) b = ceil_div(vs, ll_vecs);
        p.blocks = (int)b;
        p.cv = (int)ceil_div(vs, b);
        p.rounds = 1;
        if (c->tune_threads <= 0) {
          long long t = ((long long)p.cv + 31) / 32 * 32;
          p.threads = (int)(t < 64 ? 64 : (t > 512 ? 512 : t));
        }
        return p;
      }
    }
    const long long thr = c->oneshot_max_bytes >= 0 ? c->oneshot_max_bytes : default_oneshot_max(n);
    bool oneshot = bytes <= thr;
    if (c->tune_variant == DGN_VARIANT_ONESHOT) oneshot = true;
    if (c->tune_variant == DGN_VARIANT_TWOSHOT) oneshot = false;
    if (oneshot && ceil_div(d.nvec, bmax) > slot_vecs) oneshot = false;  // does not fit one round
    if (oneshot) {
      p.variant = DGN_VARIANT_ONESHOT;
      long long b = ceil_div(d.nvec, 512);
      if (c->tune_blocks > 0) b = c->tune_blocks;
      if (b > bmax) b = bmax;
      if (b < 1) b = 1;
      if (ceil_div(d.nvec, b) > slot_vecs) b = ceil_div(d.nvec, slot_vecs);
      p.blocks = (int)b;
      p.cv = (int)ceil_div(d.nvec, b);
      p.rounds = 1;
      return p;
    }
  }
  if (d.kind == kOpAllGather) {
    // Small blocks: flag-in-data lines, one hop.
    const long long ll_vecs = c->geo.ll_slot_bytes / 32;
    int ll_bmax = c->geo.ll_max_blocks;
    if (block_cap > 0 && block_cap < ll_bmax) ll_bmax = block_cap;
    const bool fits = ceil_div(d.nvec, ll_bmax) <= ll_vecs;
    bool ll = fits && d.nvec * 16 <= c->ll_allgather_max_bytes;
    if (c->tune_variant == DGN_VARIANT_LL) ll = fits;
    else if (c->tune_variant != DGN_VARIANT_AUTO) ll = false;
    if (ll) {
      p.variant = DGN_VARIANT_LL;
      long long b = ceil_div(d.nvec, 256);
      if (c->tune_blocks > 0) b = c->tune_blocks;
      if (b > ll_bmax) b = ll_bmax;
      if (b < 1) b = 1;
      if (ceil_div(d.nvec, b) > ll_vecs) b = ceil_div(d.nvec, ll_vecs);
      p.blocks = (int)b;
      p.cv = (int)ceil_div(d.nvec, b);
      p.rounds = 1;
      if (c->tune_threads <= 0) {
        long long t = ((long long)p.cv + 31) / 32 * 32;
        p.threads = (int)(t < 64 ? 64 : (t > 512 ? 512 : t));
      }
      return p;
    }
  }
  if (d.kind == kOpAllGather || d.kind == kOpBroadcast) {
    // Staged through the switch: a source stores its block once and the switch
    // replicates it into every rank's ring.
    if (c->nvls && !c->team) {
      const long long thr = d.kind == kOpAllGather ? c->nvls_allgather_min_bytes : c->nvls_bcast_min_bytes;
      bool nvls = d.nvec * 16 >= thr && c->tune_variant == DGN_VARIANT_AUTO;
      // Below 5 ranks the root alone through the switch wins only in the middle (4
      // ranks: 31 / 53 us against 33 / 64 us at 4 / 16 MiB, 181 against 171 us at 64 MiB).
      if (d.kind == kOpBroadcast && n < 5 && d.nvec * 16 >= c->bcast_shard_min_bytes) nvls = false;
      if (c->tune_variant == DGN_VARIANT_NVLS) nvls = true;
      if (nvls && plan_gather(c, d, block_cap, DGN_VARIANT_NVLS, &p)) return p;
    }
    // The same protocol with remote stores, or with remote loads (all-gather).
    if ((c->tune_variant == DGN_VARIANT_RING || c->tune_variant == DGN_VARIANT_RING_PULL) &&
        plan_gather(c, d, block_cap, c->tune_variant, &p))
      return p;
    if (d.kind == kOpAllGather && c->tune_variant == DGN_VARIANT_AUTO && d.nvec * 16 >= c->allgather_ring_min_bytes &&
        plan_gather(c, d, block_cap, DGN_VARIANT_RING_PULL, &p))
      return p;
  }
  // Multi-round kernels: two-shot all-reduce, reduce-scatter, all-gather,
  // broadcast.  `per` = vectors each block column has to cover.
  long long per = d.nvec;
  if (d.kind == kOpAllReduce || d.kind == kOpAllReduceUpdate) per = ceil_div(d.nvec, n);
  // Sharded optimizer step: the longest shard, ceil(total / n) elements, may
  // begin and end inside a vector.
  if (is_zero_kind(d.kind)) per = ceil_div(ceil_div(d.count, n), 16 / (long long)kElemSize[d.dtype]) + 1;
  p.variant = DGN_VARIANT_TWOSHOT;
  if (d.kind == kOpAllGather) {
    // Stores only (peers are pushed to) up to the measured crossover, pulling above.
    bool pull = d.nvec * 16 >= c->allgather_pull_min_bytes && c->tune_variant == DGN_VARIANT_AUTO;
    if (c->tune_variant == DGN_VARIANT_ONESHOT) pull = true;
    if (pull) p.variant = DGN_VARIANT_ONESHOT;
  }
  if (d.kind == kOpBroadcast) {
    // Small messages: peers pull from the root (one flag exchange).  Large
    // ones: scatter + all-gather, so the root sends about 2 S instead of
    // (n - 1) S.  With two ranks both send S and pulling is one step shorter.
    const long long thr = c->bcast_scatter_min_bytes;
    bool scatter = n > 2 && d.nvec * 16 >= thr;
    if (c->tune_variant == DGN_VARIANT_ONESHOT) scatter = false;
    if (c->tune_variant == DGN_VARIANT_TWOSHOT && n > 2) scatter = true;
    if (scatter) per = ceil_div(d.nvec, n);
    else p.variant = DGN_VARIANT_ONESHOT;
  }
  int bdef = bmax < c->num_sms ? bmax : c->num_sms;  // one block per SM
  if (c->tune_blocks > 0) bdef = bmax;
  long long b = ceil_div(per, 512);
  if (b > bdef) b = bdef;
  if (b < 1) b = 1;
  long long cv = ceil_div(per, b);
  if (cv > cv_cap) cv = cv_cap;
  if (cv < 1) cv = 1;
  p.blocks = (int)b;
  p.cv = (int)cv;
  p.rounds = (int)ceil_div(per, b * cv);
  if (p.rounds < 1) p.rounds = 1;
  return p;
}

// Geometry, wait limit and variant thresholds of a communicator of
// c->nranks ranks, from the environment and the measured defaults.  No device
// is touched.
void load_thresholds(dgn_comm* c) {
  const int nranks = c->nranks;
  c->geo = make_geometry(nranks);
  c->wait_ns = (u64)env_ll("DGN_WAIT_LIMIT_MS", 5000) * 1000000ull;
  c->oneshot_max_bytes = env_ll("DGN_ONESHOT_MAX_BYTES", -1);
  c->ll_max_bytes = env_ll("DGN_LL_MAX_BYTES", -1);
  c->ll2_max_bytes = env_ll("DGN_LL2_MAX_BYTES", -1);
  c->fused_twoshot = env_ll("DGN_TWOSHOT_FUSED", 0) != 0;
  c->bcast_scatter_min_bytes = env_ll("DGN_BCAST_SCATTER_MIN_BYTES", nranks >= 5 ? (2ll << 20) : (1ll << 20));  // 8 ranks, 1 MiB: pulling 25 us, scatter 34 us
  // Every rank receives (n - 1) * 2 * S bytes of lines: 15.7 us against 26.2 us
  // for pulling at 2 ranks and 512 KiB blocks, but no gain at 8 ranks there.
  c->ll_allgather_max_bytes =
      env_ll("DGN_LL_ALLGATHER_MAX_BYTES", nranks <= 2 ? (512ll << 10) : nranks <= 4 ? (256ll << 10) : (64ll << 10));
  // Pushing wins up to 4 MiB blocks (85 against 100 us at 8 ranks), pulling from
  // 16 MiB (222 against 246 us; 803 against 838 us at 64 MiB).
  c->allgather_pull_min_bytes = env_ll("DGN_ALLGATHER_PULL_MIN_BYTES", nranks >= 5 ? (8ll << 20) : (1ll << 62));
  c->allgather_ring_min_bytes = env_ll("DGN_ALLGATHER_RING_MIN_BYTES", 1ll << 62);
  // Shapes of the staged kernels (0: automatic).
  c->gather_chunk_bytes = env_ll("DGN_GATHER_CHUNK_BYTES", 0);
  c->gather_push_blocks = (int)env_ll("DGN_GATHER_PUSH_BLOCKS", 0);
  c->gather_forward_blocks = (int)env_ll("DGN_GATHER_FORWARD_BLOCKS", 0);
  c->gather_mode = (int)env_ll("DGN_GATHER_MODE", 0);
  c->bcast_shard_min_bytes = env_ll("DGN_BCAST_SHARD_MIN_BYTES", 32ll << 20);
  c->flow_chunk_bytes = env_ll("DGN_FLOW_CHUNK_BYTES", 0);
  c->flow_switch_blocks = (int)env_ll("DGN_FLOW_SWITCH_BLOCKS", 0);
  c->flow_in_blocks = (int)env_ll("DGN_FLOW_IN_BLOCKS", 0);
  c->flow_out_blocks = (int)env_ll("DGN_FLOW_OUT_BLOCKS", 0);
  c->flow_depth = (int)env_ll("DGN_FLOW_DEPTH", 0);
  c->unroll = (int)env_ll("DGN_NVLS_UNROLL", 0);
  c->tune_variant = (int)env_ll("DGN_FORCE_VARIANT", 0);
}

// Sizes and thresholds of the NVSwitch multicast paths; `symm_request` is the
// size of the symmetric arena asked for.  No device is touched.
void load_nvls_settings(dgn_comm* c, long long symm_request) {
  const int nranks = c->nranks;
  // Layout of the multicast-bound buffer: [ring of the staged gather (all-gather
  // and broadcast)][ring of the staged all-reduce][symmetric arena].
  const size_t gran = (size_t)2 << 20;
  long long gring = env_ll("DGN_NVLS_GATHER_RING_BYTES", (long long)nranks * (32ll << 20));
  if (gring < 0) gring = 0;
  c->gather_ring_bytes = ((size_t)gring + gran - 1) / gran * gran;
  c->nvls_bytes = c->gather_ring_bytes;
  c->flow_ring_off = (c->nvls_bytes + gran - 1) / gran * gran;
  long long ring = env_ll("DGN_NVLS_RING_BYTES", 256ll << 20);
  if (ring < 0) ring = 0;
  c->flow_ring_bytes = ((size_t)ring + gran - 1) / gran * gran;
  c->nvls_bytes = c->flow_ring_off + c->flow_ring_bytes;
  // Optional symmetric arena behind it (2 MiB granules).
  if (symm_request > 0) {
    c->symm_off = c->nvls_bytes;
    c->symm_bytes = ((size_t)symm_request + gran - 1) / gran * gran;
    c->nvls_bytes = c->symm_off + c->symm_bytes;
  }
  // Staged through the switch from this size on (any tensors, buckets included).
  // With two ranks the switch saves nothing (1.5 S per direction against 1.0 S
  // for the store-only two-shot kernel), so it is opt-in there.  Measured at 8
  // ranks against the two-shot kernel: 77 against 84 us at 16 MiB, 115 against 129
  // at 32 MiB, 189 against 227 at 64 MiB; level at 8 MiB (57 against 59).
  c->nvls_min_bytes = env_ll("DGN_NVLS_MIN_BYTES", nranks >= 8 ? (16ll << 20) : (1ll << 62));
  // In place on symmetric memory from this size on; never by default at two
  // ranks (measured there: 401 GB/s against 577 GB/s for two-shot at 256 MiB).
  c->symm_min_bytes = env_ll("DGN_SYMM_MIN_BYTES", nranks <= 2 ? (1ll << 62) : (4ll << 20));
  // Through the switch the root sends S bytes whatever the rank count.  Measured
  // at 8 ranks: peers pulling from the root is level up to 1 MiB (22 to 25 us) and
  // falls behind above (56 us at 4 MiB against 34 us staged through the switch and
  // 38 us for scatter + all-gather by remote stores; 66 / 73 us at 16 MiB; 181 /
  // 201 us at 64 MiB).  At 3 and 4 ranks it is used from 4 MiB to below 32 MiB; at 2
  // ranks the switch loses (178 against 118 us at 64 MiB), so it is opt-in there.
  c->nvls_bcast_min_bytes = env_ll("DGN_NVLS_BCAST_MIN_BYTES", nranks >= 5 ? (2ll << 20) : nranks >= 3 ? (4ll << 20) : (1ll << 62));
  c->nvls_allgather_min_bytes = env_ll("DGN_NVLS_ALLGATHER_MIN_BYTES", 1ll << 62);
}

struct KernelChoice {
  const void* fn = nullptr;
  size_t smem = 0;
};

KernelChoice choose_kernel(const dgn_comm* c, const OpDesc& d, const Plan& p) {
  KernelChoice k;
  const bool table = d.ntensors > 1;
  switch (d.kind) {
    case kOpAllReduce:
      k.fn = reduce_fn(d.dtype, p.variant == DGN_VARIANT_RING ? 8 : p.variant == DGN_VARIANT_SYMM ? 7 : p.variant == DGN_VARIANT_NVLS ? 6 : p.variant == DGN_VARIANT_LL2 ? 5 : p.variant == DGN_VARIANT_LL ? 3 : (p.variant == DGN_VARIANT_ONESHOT ? 0 : (p.threads >= 96 && p.rounds >= 3 && !c->fused_twoshot ? 4 : 1)), table);
      k.smem = table ? table_smem_bytes(d.ntensors) : 0;
      break;
    case kOpReduceScatter: k.fn = reduce_fn(d.dtype, 2, false); break;
    case kOpAllGather:
      k.fn = p.variant == DGN_VARIANT_NVLS      ? gather_flow_kernel_fn(true)
             : p.variant == DGN_VARIANT_RING || p.variant == DGN_VARIANT_RING_PULL ? gather_flow_kernel_fn(false)
             : p.variant == DGN_VARIANT_LL      ? allgather_ll_kernel_fn()
             : p.variant == DGN_VARIANT_ONESHOT ? allgather_pull_kernel_fn()
                                                : allgather_kernel_fn();
      break;
    case kOpBroadcast:
      k.fn = p.variant == DGN_VARIANT_NVLS      ? gather_flow_kernel_fn(true)
             : p.variant == DGN_VARIANT_RING    ? gather_flow_kernel_fn(false)
             : p.variant == DGN_VARIANT_TWOSHOT ? broadcast_scatter_kernel_fn()
                                                : broadcast_kernel_fn();
      break;
    case kOpAllReduceUpdate:
      k.fn = update_kernel_fn(d.uh.kind);
      k.smem = update_smem_bytes(d.ntensors);
      break;
    case kOpZeroReduce:
    case kOpZeroUpdate:
      k.fn = zero_kernel_fn(d.dtype, d.kind == kOpZeroReduce ? 0 : 1);
      k.smem = zero_smem_bytes(d.ntensors);
      break;
  }
  return k;
}

void fill_params(OpParams* P, const dgn_comm* c, const OpDesc& d, const Plan& p) {
  memset(P, 0, sizeof(*P));
  P->count = d.count;
  P->nvec = d.nvec;
  P->wait_ns = c->wait_ns;
  P->scale = (double)(1.f / (float)c->nranks);
  P->ntensors = d.ntensors;
  P->rounds = p.rounds;
  P->cv = p.cv;
  P->redop = d.redop;
  P->root = d.kind == kOpAllGather ? -1 : d.root;  // staged gather: every rank is a source
  P->unroll = p.unroll;
  P->pattern = c->pattern;
  P->flow_cv = p.cv;
  P->flow_chunks = p.rounds;
  P->flow_depth = p.flow_depth;
  P->flow_nsw = p.flow_nsw;
  P->flow_nin = p.flow_nin;
  P->flow_mode = p.flow_mode;
  P->inbox_off = p.inbox_off;
}

void fill_zero_params(ZeroParams* Z, const dgn_comm* c, const OpDesc& d, const Plan& p) {
  memset(Z, 0, sizeof(*Z));
  fill_params(&Z->base, c, d, p);
  Z->total = d.count;
  Z->rc = ceil_div(d.count, c->nranks);
  Z->lr = d.zh.lr;
  Z->beta1 = d.zh.beta1;
  Z->beta2 = d.zh.beta2;
  Z->eps = d.zh.eps;
  Z->wd = d.zh.wd;
  Z->grad_scale = d.zh.grad_scale;
  Z->clip_norm = d.zh.clip_norm;
  Z->clip_value = d.zh.clip_value;
  Z->check_finite = d.zh.check_finite;
  Z->use_lr_scales = d.zh.use_lr_scales;
}

void fill_update_params(UpdParams* U, const dgn_comm* c, const OpDesc& d, const Plan& p) {
  memset(U, 0, sizeof(*U));
  fill_params(&U->base, c, d, p);
  U->kind = d.uh.kind;
  U->lr = d.uh.lr;
  U->a = d.uh.a;
  U->b = d.uh.b;
  U->eps = d.uh.eps;
  U->wd = d.uh.wd;
  U->grad_scale = d.uh.grad_scale;
  U->clip_value = d.uh.clip_value;
}

int launch(const void* fn, dim3 grid, int threads, size_t smem, cudaStream_t stream, void* P,
           bool cooperative) {
  void* args[1] = {P};
  cudaError_t e = cooperative
                      ? cudaLaunchCooperativeKernel(fn, grid, dim3(threads), args, smem, stream)
                      : cudaLaunchKernel(fn, grid, dim3(threads), args, smem, stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(DGN_ERR_CUDA, "kernel launch failed: %s (grid %u x %u, %d threads, %zu B smem)",
                cudaGetErrorString(e), grid.x, grid.y, threads, smem);
  }
  g_launches.fetch_add(1);
  return DGN_OK;
}

int check_ready(dgn_comm* c) {
  if (!c) return fail(DGN_ERR_ARG, "null communicator");
  if (!c->connected) return fail(DGN_ERR_STATE, "communicator is not connected");
  if (c->status_host && *c->status_host != 0)
    return fail(DGN_ERR_STATE, "communicator is unusable: an earlier collective reported status %d (%s)",
                *c->status_host, dgn_status_string(*c->status_host));
  return DGN_OK;
}

// Issues one multi-rank collective: directly for a real rank, or once every
// virtual rank of an emulated team has arrived.
int issue(dgn_comm* c, const OpDesc& d) {
  DeviceGuard g(c->device);
  c->last_stream = d.stream;
  c->has_last_stream = true;
  if (!c->team) {
    Plan p = make_plan(c, d, 0);
    KernelChoice k = choose_kernel(c, d, p);
    if (!k.fn) return fail(DGN_ERR_UNSUPPORTED, "no kernel for dtype %d", d.dtype);
    int rc;
    if ((d.kind == kOpAllReduce || d.kind == kOpAllGather || d.kind == kOpBroadcast) &&
        (p.variant == DGN_VARIANT_NVLS || p.variant == DGN_VARIANT_RING || p.variant == DGN_VARIANT_RING_PULL)) {
      // The blocks of the dataflow kernels wait for one another: cooperative launch.
      OpParams P;
      fill_params(&P, c, d, p);
      P.peers[0] = c->table;
      P.ra[0].in = d.in;
      P.ra[0].out = d.out;
      P.ra[0].table = d.table;
      rc = launch(k.fn, dim3(p.blocks, 1), p.threads, k.smem, d.stream, &P, true);
    } else if (is_zero_kind(d.kind)) {
      ZeroParams Z;
      fill_zero_params(&Z, c, d, p);
      Z.base.peers[0] = c->table;
      Z.zr[0] = d.zr;
      rc = launch(k.fn, dim3(p.blocks, 1), p.threads, k.smem, d.stream, &Z, false);
    } else if (d.kind == kOpAllReduceUpdate) {
      UpdParams U;
      fill_update_params(&U, c, d, p);
      U.base.peers[0] = c->table;
      U.table[0] = d.utable;
      rc = launch(k.fn, dim3(p.blocks, 1), p.threads, k.smem, d.stream, &U, false);
    } else {
      OpParams P;
      fill_params(&P, c, d, p);
      P.peers[0] = c->table;
      P.ra[0].in = d.in;
      P.ra[0].out = d.out;
      P.ra[0].table = d.table;
      rc = launch(k.fn, dim3(p.blocks, 1), p.threads, k.smem, d.stream, &P, false);
    }
    if (rc != DGN_OK) return rc;
    c->last_plan = p;
    return DGN_OK;
  }
  // Emulated team: a virtual rank may run several collectives ahead of the
  // others (one operator call can issue one per bucket), so calls queue per
  // rank; whenever every rank has one waiting, the heads are launched together.
  Team* t = c->team;
  t->pending[c->rank].push_back(d);
  for (;;) {
    for (int r = 0; r < t->n; ++r)
      if (t->pending[r].empty()) return DGN_OK;
    const OpDesc f = t->pending[0].front();
    for (int r = 1; r < t->n; ++r) {
      const OpDesc& o = t->pending[r].front();
      if (f.kind != o.kind || f.dtype != o.dtype || f.redop != o.redop || f.root != o.root ||
          f.count != o.count || f.nvec != o.nvec || f.ntensors != o.ntensors || f.stream != o.stream ||
          memcmp(&f.zh, &o.zh, sizeof(ZeroHyper)) != 0 || memcmp(&f.uh, &o.uh, sizeof(UpdHyper)) != 0) {
        for (int q = 0; q < t->n; ++q) t->pending[q].clear();
        return fail(DGN_ERR_ARG, "virtual rank %d issued a collective that differs from rank 0's", r);
      }
    }
    // Shape the launch so that every block of every virtual rank is resident.
    // A smaller grid can mean another block size, hence another occupancy:
    // iterate until the plan fits its own cap.
    Plan p = make_plan(c, f, 0);
    KernelChoice k = choose_kernel(c, f, p);
    bool fits = false;
    for (int iter = 0; iter < 6 && !fits; ++iter) {
      if (!k.fn) return fail(DGN_ERR_UNSUPPORTED, "no kernel for dtype %d", f.dtype);
      int per_sm = 0;
      DGN_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k.fn, p.threads, k.smem));
      const int cap = per_sm * c->num_sms / t->n;
      if (cap < 1) return fail(DGN_ERR_UNSUPPORTED, "emulated team does not fit on the device");
      if (p.blocks <= cap) {
        fits = true;
      } else {
        p = make_plan(c, f, cap);
        k = choose_kernel(c, f, p);
      }
    }
    if (!fits) return fail(DGN_ERR_UNSUPPORTED, "no resident launch shape for the emulated team");
    OpParams P;
    ZeroParams Z;
    UpdParams U;
    const bool zero = is_zero_kind(f.kind), upd = f.kind == kOpAllReduceUpdate;
    if (zero) fill_zero_params(&Z, c, f, p);
    else if (upd) fill_update_params(&U, c, f, p);
    else fill_params(&P, c, f, p);
    for (int r = 0; r < t->n; ++r) {
      const OpDesc& o = t->pending[r].front();
      if (zero) {
        Z.base.peers[r] = t->members[r]->table;
        Z.zr[r] = o.zr;
      } else if (upd) {
        U.base.peers[r] = t->members[r]->table;
        U.table[r] = o.utable;
      } else {
        P.peers[r] = t->members[r]->table;
        P.ra[r].in = o.in;
        P.ra[r].out = o.out;
        P.ra[r].table = o.table;
      }
    }
    for (int r = 0; r < t->n; ++r) t->pending[r].pop_front();
    int rc = launch(k.fn, dim3(p.blocks, t->n), p.threads, k.smem, f.stream,
                    zero ? (void*)&Z : upd ? (void*)&U : (void*)&P, true);
    if (rc != DGN_OK) return rc;
    for (dgn_comm* m : t->members) m->last_plan = p;
  }
}

int launch_local_copy(dgn_comm* c, const OpDesc& d, int es) {
  DeviceGuard g(c->device);
  const bool table = d.ntensors > 1;
  const void* fn = local_copy_kernel_fn(es, table);
  if (!fn) return fail(DGN_ERR_UNSUPPORTED, "no copy kernel for element size %d", es);
  Plan p;
  // Measured on B200 (256 MiB and 1 GiB copies): 256 threads and 32 blocks per
  // SM reach the bandwidth of a device-to-device memcpy; fewer, larger blocks
  // lose 5-10 %.
  p.threads = c->tune_threads > 0 ? c->tune_threads : 256;
  if (p.threads > kMaxThreads) p.threads = kMaxThreads;
  long long b = ceil_div(d.nvec, (long long)p.threads * 4);
  const long long cap = c->tune_blocks > 0 ? c->tune_blocks : (long long)c->num_sms * 32;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  p.blocks = (int)b;
  p.variant = 0;
  OpParams P;
  fill_params(&P, c, d, p);
  P.ra[0].in = d.in;
  P.ra[0].out = d.out;
  P.ra[0].table = d.table;
  int rc = launch(fn, dim3(p.blocks, 1), p.threads, table ? table_smem_bytes(d.ntensors) : 0,
                  d.stream, &P, false);
  if (rc == DGN_OK) c->last_plan = p;
  return rc;
}

// Device table for a bucket of tensors, cached on the tensor list (the same
// gradients come back every step).
int get_table(dgn_comm* c, const void* const* in, void* const* out, const int64_t* counts, int nt,
              int es, cudaStream_t stream, const TableEntry** result) {
  for (TableEntry& e : c->tables) {
    if (e.es == es && (int)e.in.size() == nt && memcmp(e.in.data(), in, sizeof(void*) * nt) == 0 &&
        memcmp(e.out.data(), out, sizeof(void*) * nt) == 0 &&
        memcmp(e.counts.data(), counts, sizeof(int64_t) * nt) == 0) {
      e.last_use = ++c->table_clock;
      // A call on another stream than the one that uploaded the table must not overtake the upload.
      if (stream != e.upload_stream && e.uploaded) DGN_CUDA(cudaStreamWaitEvent(stream, e.uploaded, 0));
      *result = &e;
      return DGN_OK;
    }
  }
  // Evict the least recently used entry -- unless calls of this virtual rank
  // are still queued: they hold table pointers that are not on the device yet.
  if (c->tables.size() >= 32 && !(c->team && !c->team->pending[c->rank].empty())) {
    size_t lru = 0;
    for (size_t i = 1; i < c->tables.size(); ++i)
      if (c->tables[i].last_use < c->tables[lru].last_use) lru = i;
    cudaFree(c->tables[lru].d_table);  // synchronises with any kernel still reading it
    cudaFreeHost(c->tables[lru].h_table);
    if (c->tables[lru].uploaded) cudaEventDestroy(c->tables[lru].uploaded);
    c->tables.erase(c->tables.begin() + lru);
  }
  TableEntry e;
  e.es = es;
  e.in.assign(in, in + nt);
  e.out.assign(out, out + nt);
  e.counts.assign(counts, counts + nt);
  DGN_CUDA(cudaHostAlloc((void**)&e.h_table, sizeof(TensorEnt) * (size_t)(nt + 1), cudaHostAllocDefault));
  long long v = 0;
  int k = 0;
  for (int i = 0; i < nt; ++i) {
    if (counts[i] == 0) continue;
    e.h_table[k].in = static_cast<const char*>(in[i]);
    e.h_table[k].out = static_cast<char*>(out[i]);
    e.h_table[k].count = counts[i];
    e.h_table[k].vbegin = v;
    v += ceil_div(counts[i] * es, 16);
    ++k;
  }
  e.nt = k;
  e.nvec = v;
  cudaError_t err = cudaMalloc((void**)&e.d_table, sizeof(TensorEnt) * (size_t)(nt + 1));
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(e.d_table, e.h_table, sizeof(TensorEnt) * (size_t)k, cudaMemcpyHostToDevice, stream);
  if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e.uploaded, cudaEventDisableTiming);
  if (err == cudaSuccess) err = cudaEventRecord(e.uploaded, stream);
  if (err != cudaSuccess) {
    cudaFree(e.d_table);
    cudaFreeHost(e.h_table);
    if (e.uploaded) cudaEventDestroy(e.uploaded);
    return fail(DGN_ERR_CUDA, "bucket table: %s", cudaGetErrorString(err));
  }
  e.upload_stream = stream;
  e.last_use = ++c->table_clock;
  c->tables.push_back(std::move(e));
  *result = &c->tables.back();
  return DGN_OK;
}

// Device table of a sharded optimizer step (gradients, parameters, flat
// element offsets, learning-rate scales), cached like the bucket tables.
int get_zero_table(dgn_comm* c, const void* const* grads, void* const* params, const int64_t* counts, int nt,
                   const float* lrs, int es, cudaStream_t stream, const ZeroTableEntry** result) {
  for (ZeroTableEntry& e : c->zero_tables) {
    if (e.es == es && (int)e.grads.size() == nt && memcmp(e.grads.data(), grads, sizeof(void*) * nt) == 0 &&
        memcmp(e.params.data(), params, sizeof(void*) * nt) == 0 &&
        memcmp(e.counts.data(), counts, sizeof(int64_t) * nt) == 0 &&
        (lrs ? (e.lrs.size() == (size_t)nt && memcmp(e.lrs.data(), lrs, sizeof(float) * nt) == 0) : e.lrs.empty())) {
      e.last_use = ++c->table_clock;
      if (stream != e.upload_stream && e.uploaded) DGN_CUDA(cudaStreamWaitEvent(stream, e.uploaded, 0));
      *result = &e;
      return DGN_OK;
    }
  }
  if (c->zero_tables.size() >= 16 && !(c->team && !c->team->pending[c->rank].empty())) {  // as above
    size_t lru = 0;
    for (size_t i = 1; i < c->zero_tables.size(); ++i)
      if (c->zero_tables[i].last_use < c->zero_tables[lru].last_use) lru = i;
    cudaFree(c->zero_tables[lru].d_table);  // synchronises with any kernel still reading it
    cudaFreeHost(c->zero_tables[lru].h_table);
    if (c->zero_tables[lru].uploaded) cudaEventDestroy(c->zero_tables[lru].uploaded);
    c->zero_tables.erase(c->zero_tables.begin() + lru);
  }
  ZeroTableEntry e;
  e.es = es;
  e.grads.assign(grads, grads + nt);
  e.params.assign(params, params + nt);
  e.counts.assign(counts, counts + nt);
  if (lrs) e.lrs.assign(lrs, lrs + nt);
  DGN_CUDA(cudaHostAlloc((void**)&e.h_table, sizeof(ZeroEnt) * (size_t)(nt + 1), cudaHostAllocDefault));
  long long total = 0;
  int k = 0;
  for (int i = 0; i < nt; ++i) {
    if (counts[i] == 0) continue;
    e.h_table[k].grad = static_cast<const char*>(grads[i]);
    e.h_table[k].param = static_cast<char*>(params[i]);
    e.h_table[k].ebegin = total;
    e.h_table[k].lr_scale = lrs ? lrs[i] : 1.f;
    e.h_table[k].reserved = 0;
    total += counts[i];
    ++k;
  }
  e.nt = k;
  e.total = total;
  cudaError_t err = cudaMalloc((void**)&e.d_table, sizeof(ZeroEnt) * (size_t)(nt + 1));
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(e.d_table, e.h_table, sizeof(ZeroEnt) * (size_t)k, cudaMemcpyHostToDevice, stream);
  if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e.uploaded, cudaEventDisableTiming);
  if (err == cudaSuccess) err = cudaEventRecord(e.uploaded, stream);
  if (err != cudaSuccess) {
    cudaFree(e.d_table);
    cudaFreeHost(e.h_table);
    if (e.uploaded) cudaEventDestroy(e.uploaded);
    return fail(DGN_ERR_CUDA, "bucket table of the sharded optimizer step: %s", cudaGetErrorString(err));
  }
  e.upload_stream = stream;
  e.last_use = ++c->table_clock;
  c->zero_tables.push_back(std::move(e));
  *result = &c->zero_tables.back();
  return DGN_OK;
}

// Device table of an all-reduce fused with the optimizer update, cached like the bucket tables.
int get_update_table(dgn_comm* c, const void* const* grads, void* const* params, void* const* m, void* const* v,
                     const int64_t* counts, int nt, cudaStream_t stream, const UpdTableEntry** result) {
  for (UpdTableEntry& e : c->upd_tables) {
    if ((int)e.grads.size() == nt && memcmp(e.grads.data(), grads, sizeof(void*) * nt) == 0 &&
        memcmp(e.params.data(), params, sizeof(void*) * nt) == 0 && memcmp(e.m.data(), m, sizeof(void*) * nt) == 0 &&
        (v ? (e.v.size() == (size_t)nt && memcmp(e.v.data(), v, sizeof(void*) * nt) == 0) : e.v.empty()) &&
        memcmp(e.counts.data(), counts, sizeof(int64_t) * nt) == 0) {
      e.last_use = ++c->table_clock;
      if (stream != e.upload_stream && e.uploaded) DGN_CUDA(cudaStreamWaitEvent(stream, e.uploaded, 0));
      *result = &e;
      return DGN_OK;
    }
  }
  if (c->upd_tables.size() >= 16 && !(c->team && !c->team->pending[c->rank].empty())) {
    size_t lru = 0;
    for (size_t i = 1; i < c->upd_tables.size(); ++i)
      if (c->upd_tables[i].last_use < c->upd_tables[lru].last_use) lru = i;
    cudaFree(c->upd_tables[lru].d_table);  // synchronises with any kernel still reading it
    cudaFreeHost(c->upd_tables[lru].h_table);
    if (c->upd_tables[lru].uploaded) cudaEventDestroy(c->upd_tables[lru].uploaded);
    c->upd_tables.erase(c->upd_tables.begin() + lru);
  }
  UpdTableEntry e;
  e.grads.assign(grads, grads + nt);
  e.params.assign(params, params + nt);
  e.m.assign(m, m + nt);
  if (v) e.v.assign(v, v + nt);
  e.counts.assign(counts, counts + nt);
  DGN_CUDA(cudaHostAlloc((void**)&e.h_table, sizeof(UpdEnt) * (size_t)(nt + 1), cudaHostAllocDefault));
  long long vec = 0;
  int k = 0;
  for (int i = 0; i < nt; ++i) {
    if (counts[i] == 0) continue;
    e.h_table[k].grad = static_cast<const char*>(grads[i]);
    e.h_table[k].param = static_cast<char*>(params[i]);
    e.h_table[k].m = static_cast<char*>(m[i]);
    e.h_table[k].v = v ? static_cast<char*>(v[i]) : nullptr;
    e.h_table[k].count = counts[i];
    e.h_table[k].vbegin = vec;
    vec += ceil_div(counts[i] * 4, 16);
    ++k;
  }
  e.nt = k;
  e.nvec = vec;
  cudaError_t err = cudaMalloc((void**)&e.d_table, sizeof(UpdEnt) * (size_t)(nt + 1));
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(e.d_table, e.h_table, sizeof(UpdEnt) * (size_t)k, cudaMemcpyHostToDevice, stream);
  if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e.uploaded, cudaEventDisableTiming);
  if (err == cudaSuccess) err = cudaEventRecord(e.uploaded, stream);
  if (err != cudaSuccess) {
    cudaFree(e.d_table);
    cudaFreeHost(e.h_table);
    if (e.uploaded) cudaEventDestroy(e.uploaded);
    return fail(DGN_ERR_CUDA, "table of the fused update: %s", cudaGetErrorString(err));
  }
  e.upload_stream = stream;
  e.last_use = ++c->table_clock;
  c->upd_tables.push_back(std::move(e));
  *result = &c->upd_tables.back();
  return DGN_OK;
}

// Argument checks shared by the entry points of the sharded optimizer step.
int check_zero_bucket(const void* const* a, const void* const* b, const int64_t* counts, int ntensors, int dtype,
                      long long* total, int* nonempty) {
  if (dtype != DGN_F16 && dtype != DGN_BF16 && dtype != DGN_F32)
    return fail(DGN_ERR_UNSUPPORTED, "the sharded optimizer step takes float16, bfloat16 or float32, got dtype %d", dtype);
  if (ntensors < 1 || !a || !b || !counts) return fail(DGN_ERR_ARG, "null or empty tensor list");
  const size_t es = kElemSize[dtype];
  *total = 0;
  *nonempty = 0;
  for (int i = 0; i < ntensors; ++i) {
    if (counts[i] < 0) return fail(DGN_ERR_ARG, "negative count for tensor %d", i);
    if (counts[i] == 0) continue;
    if (!a[i] || !b[i]) return fail(DGN_ERR_ARG, "null pointer for tensor %d", i);
    if (((uintptr_t)a[i] | (uintptr_t)b[i]) & (es - 1))
      return fail(DGN_ERR_ARG, "tensor %d is not aligned to its element size", i);
    *total += counts[i];
    ++*nonempty;
  }
  if (*nonempty > kMaxTableTensors)
    return fail(DGN_ERR_UNSUPPORTED, "a bucket takes at most %d tensors, got %d", kMaxTableTensors, *nonempty);
  return DGN_OK;
}

void free_comm(dgn_comm* c) {
  DeviceGuard g(c->device);
  cudaDeviceSynchronize();
  for (TableEntry& e : c->tables) {
    cudaFree(e.d_table);
    cudaFreeHost(e.h_table);
    if (e.uploaded) cudaEventDestroy(e.uploaded);
  }
  for (ZeroTableEntry& e : c->zero_tables) {
    cudaFree(e.d_table);
    cudaFreeHost(e.h_table);
    if (e.uploaded) cudaEventDestroy(e.uploaded);
  }
  for (UpdTableEntry& e : c->upd_tables) {
    cudaFree(e.d_table);
    cudaFreeHost(e.h_table);
    if (e.uploaded) cudaEventDestroy(e.uploaded);
  }
  for (int j = 0; j < c->nranks; ++j)
    if (j != c->rank && c->peer_ipc[j] && c->peer_base[j]) cudaIpcCloseMemHandle(c->peer_base[j]);
  if (c->nvls) nvls_destroy(c->nvls);
  {
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    registry().erase((uint64_t)(uintptr_t)c->base);
  }
  if (c->base) cudaFree(c->base);
  if (c->status_host) cudaFreeHost(c->status_host);
  if (c->host_pin) cudaFreeHost(c->host_pin);
  if (c->host_dev) cudaFree(c->host_dev);
  if (c->host_stream) cudaStreamDestroy(c->host_stream);
  if (!c->rdv_ok_file.empty()) unlink(c->rdv_ok_file.c_str());
  delete c;
}

bool write_file_atomic(const std::string& path, const void* data, size_t n) {
  std::string tmp = path + ".tmp";
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) return false;
  bool ok = fwrite(data, 1, n, f) == n;
  ok = (fclose(f) == 0) && ok;
  if (ok) ok = rename(tmp.c_str(), path.c_str()) == 0;
  return ok;
}

bool read_file_exact(const std::string& path, void* data, size_t n) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  bool ok = fread(data, 1, n, f) == n;
  fclose(f);
  return ok;
}

double now_s() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

}  // namespace

namespace dgn {
// For the other translation units of the library: record an error message for
// dgn_last_error_string and hand back `code`.
int report_error(int code, const char* message) { return fail(code, "%s", message); }
}  // namespace dgn

// Sets up the NVSwitch multicast staging if every rank can take part: all
// ranks in this process (the last one to connect does the work for all), or
// every rank in a process of its own (rank 0 coordinates over a socket).
// Every rank takes the same decisions from the same handle table, and the
// socket protocol makes all ranks succeed or fail together, so the variant is
// either available on all ranks or on none.  Failure is not an error: the
// communicator simply has no multicast variant.
namespace {
void drop_nvls(dgn_comm* c) {
  if (c->nvls) nvls_destroy(c->nvls);
  c->nvls = nullptr;
}

void setup_nvls(dgn_comm* c, const void* all_handles) {
  std::vector<Handle> hs(c->nranks);
  bool all_capable = true, same_pid = true, distinct_pid = true;
  for (int j = 0; j < c->nranks; ++j) {
    memcpy(&hs[j], static_cast<const char*>(all_handles) + (size_t)j * DGN_HANDLE_BYTES, sizeof(Handle));
    all_capable = all_capable && hs[j].nvls_capable != 0;
    same_pid = same_pid && hs[j].pid == hs[0].pid;
    for (int q = 0; q < j; ++q) distinct_pid = distinct_pid && hs[q].pid != hs[j].pid;
  }
  if (!all_capable || (!same_pid && !distinct_pid)) {
    drop_nvls(c);
    return;
  }
  std::string why;
  if (distinct_pid) {
    DeviceGuard g(c->device);
    int rc;
    if (c->rank == 0) {
      rc = c->nvls ? nvls_root_finish(c->nvls, 20000, &why) : 1;
      if (rc != 0) drop_nvls(c);
    } else {
      rc = nvls_peer_join(c->device, c->nranks, c->nvls_bytes, hs[0].nvls_sock, 20000, &c->nvls, &why);
      if (rc != 0) c->nvls = nullptr;
    }
    return;
  }
  // One process: wait until every member has connected, then set all up at once.
  std::lock_guard<std::mutex> lock(g_registry_mutex);
  std::vector<dgn_comm*> members(c->nranks, nullptr);
  for (int j = 0; j < c->nranks; ++j) {
    auto it = registry().find(hs[j].base_ptr);
    if (it == registry().end()) return;
    members[j] = it->second;
    if (members[j] != c && !members[j]->connected) return;  // not the last one yet
  }
  drop_nvls(members[0]);  // the socket-mode preparation of rank 0 is not needed here
  std::vector<int> devices(c->nranks);
  for (int j = 0; j < c->nranks; ++j) devices[j] = members[j]->device;
  std::vector<NvlsBuffer*> bufs(c->nranks, nullptr);
  if (nvls_setup_inprocess(c->nranks, devices.data(), c->nvls_bytes, bufs.data(), &why) != 0) return;
  for (int j = 0; j < c->nranks; ++j) {
    members[j]->nvls = bufs[j];
    if (members[j] != c) fill_peer_table(members[j], &members[j]->table);
  }
}
}  // namespace

// ---------------------------------------------------------------------------
// C-ABI

extern "C" {

int dgn_version(void) { return 100; }

size_t dgn_dtype_size(int dtype) { return (dtype >= 0 && dtype < 8) ? kElemSize[dtype] : 0; }

const char* dgn_last_error_string(void) { return g_err; }

const char* dgn_status_string(int status) {
  switch (status) {
    case DGN_OK: return "ok";
    case DGN_ERR_ARG: return "invalid argument";
    case DGN_ERR_CUDA: return "CUDA error";
    case DGN_ERR_TIMEOUT: return "timed out waiting for a peer";
    case DGN_ERR_PEER: return "peer not reachable";
    case DGN_ERR_STATE: return "invalid state";
    case DGN_ERR_UNSUPPORTED: return "unsupported";
    default: return "unknown status";
  }
}

int dgn_comm_init_local(int rank, int nranks, int device, dgn_comm_t* comm) {
  if (!comm) return fail(DGN_ERR_ARG, "comm is null");
  *comm = nullptr;
  if (nranks < 1 || nranks > DGN_MAX_RANKS) return fail(DGN_ERR_ARG, "nranks %d outside 1..%d", nranks, DGN_MAX_RANKS);
  if (rank < 0 || rank >= nranks) return fail(DGN_ERR_ARG, "rank %d outside 0..%d", rank, nranks - 1);
  int ndev = 0;
  DGN_CUDA(cudaGetDeviceCount(&ndev));
  if (device < 0 || device >= ndev) return fail(DGN_ERR_ARG, "device %d outside 0..%d", device, ndev - 1);
  dgn_comm* c = new dgn_comm();
  c->rank = rank;
  c->nranks = nranks;
  c->device = device;
  {
    struct timespec ts;
    clock_gettime(CLOCK_REALTIME, &ts);
    c->session = ((uint64_t)getpid() << 40) ^ ((uint64_t)ts.tv_sec << 20) ^ (uint64_t)ts.tv_nsec ^ (uint64_t)rank;
  }
  load_thresholds(c);
  int rc = alloc_workspace(c);
  if (rc != DGN_OK) {
    free_comm(c);
    return rc;
  }
  {
    std::lock_guard<std::mutex> lock(g_registry_mutex);
    registry()[(uint64_t)(uintptr_t)c->base] = c;
  }
  if (nranks > 1 && !g_skip_nvls && env_ll("DGN_NVLS", 1) != 0) {
    DeviceGuard g(device);
    load_nvls_settings(c, g_symm_request >= 0 ? g_symm_request : env_ll("DGN_SYMM_BYTES", 0));
    c->nvls_capable = nvls_device_supported(device);
    if (c->nvls_capable && rank == 0) {
      // Rank 0 owns the multicast object and the rendezvous socket.
      std::string why;
      if (nvls_root_prepare(device, nranks, c->nvls_bytes, &c->nvls, c->nvls_sock, &why) != 0) {
        c->nvls = nullptr;
        c->nvls_capable = false;
      }
    }
  }
  if (nranks == 1) {
    c->peer_base[0] = c->base;
    fill_peer_table(c, &c->table);
    c->connected = true;
  }
  *comm = c;
  return DGN_OK;
}

int dgn_comm_init_symmetric(int rank, int nranks, int device, int64_t symm_bytes, dgn_comm_t* comm) {
  if (symm_bytes < 0) return fail(DGN_ERR_ARG, "negative arena size");
  g_symm_request = symm_bytes;
  const int rc = dgn_comm_init_local(rank, nranks, device, comm);
  g_symm_request = -1;
  return rc;
}

int64_t dgn_comm_symm_capacity(dgn_comm_t c) { return (c && c->nvls) ? (int64_t)c->symm_bytes : 0; }

int dgn_comm_symm_alloc(dgn_comm_t c, int64_t bytes, void** ptr) {
  if (!c || !ptr || bytes < 0) return fail(DGN_ERR_ARG, "bad argument");
  *ptr = nullptr;
  if (!c->connected) return fail(DGN_ERR_STATE, "communicator is not connected");
  if (!c->nvls || c->symm_bytes == 0)
    return fail(DGN_ERR_UNSUPPORTED, "this communicator has no symmetric arena (no NVSwitch multicast, or size 0)");
  const size_t need = ((size_t)bytes + 255) & ~(size_t)255;
  if (c->symm_used + need > c->symm_bytes)
    return fail(DGN_ERR_ARG, "symmetric arena exhausted: %zu of %zu bytes in use, %zu requested", c->symm_used,
                c->symm_bytes, need);
  char *uc = nullptr, *mc = nullptr;
  nvls_pointers(c->nvls, &uc, &mc);
  *ptr = uc + c->symm_off + c->symm_used;
  c->symm_used += need;
  return DGN_OK;
}

int dgn_comm_symm_reset(dgn_comm_t c) {
  if (!c) return fail(DGN_ERR_ARG, "null communicator");
  c->symm_used = 0;
  return DGN_OK;
}

int dgn_comm_get_handle(dgn_comm_t c, void* handle) {
  if (!c || !handle) return fail(DGN_ERR_ARG, "null argument");
  DeviceGuard g(c->device);
  Handle h;
  memset(&h, 0, sizeof(h));
  h.magic = kMagic;
  h.version = (uint32_t)dgn_version();
  h.pid = (int32_t)getpid();
  h.device = c->device;
  h.rank = c->rank;
  h.nranks = c->nranks;
  h.max_blocks = c->geo.max_blocks;
  h.slot_bytes = c->geo.slot_bytes;
  h.total_bytes = c->geo.total;
  h.base_ptr = (uint64_t)(uintptr_t)c->base;
  h.host_id = host_identity();
  DGN_CUDA(cudaIpcGetMemHandle(&h.ipc, c->base));
  h.nvls_capable = c->nvls_capable ? 1 : 0;
  memcpy(h.nvls_sock, c->nvls_sock, sizeof(h.nvls_sock));
  h.symm_bytes = c->symm_bytes;
  h.session = c->session;
  memset(handle, 0, DGN_HANDLE_BYTES);
  memcpy(handle, &h, sizeof(h));
  return DGN_OK;
}

int dgn_comm_connect(dgn_comm_t c, const void* all_handles) {
  if (!c || !all_handles) return fail(DGN_ERR_ARG, "null argument");
  if (c->team) return fail(DGN_ERR_STATE, "emulated communicators are connected at creation");
  if (c->connected && c->nranks > 1) return fail(DGN_ERR_STATE, "already connected");
  DeviceGuard g(c->device);
  const uint64_t me_host = host_identity();
  const int32_t me_pid = (int32_t)getpid();
  for (int j = 0; j < c->nranks; ++j) {
    Handle h;
    memcpy(&h, static_cast<const char*>(all_handles) + (size_t)j * DGN_HANDLE_BYTES, sizeof(h));
    if (h.magic != kMagic || h.version != (uint32_t)dgn_version())
      return fail(DGN_ERR_ARG, "handle %d is not a dgn handle of this version", j);
    if (h.rank != j || h.nranks != c->nranks)
      return fail(DGN_ERR_ARG, "handle %d describes rank %d of %d", j, h.rank, h.nranks);
    if (h.max_blocks != c->geo.max_blocks || h.slot_bytes != c->geo.slot_bytes || h.total_bytes != c->geo.total)
      return fail(DGN_ERR_ARG, "rank %d uses a different workspace geometry", j);
    if (h.symm_bytes != c->symm_bytes)
      return fail(DGN_ERR_ARG, "rank %d asked for a symmetric arena of %llu bytes, this rank for %zu", j,
                  (unsigned long long)h.symm_bytes, c->symm_bytes);
    if (h.host_id != me_host) return fail(DGN_ERR_PEER, "rank %d is on another host", j);
    if (j == c->rank) {
      c->peer_base[j] = c->base;
      continue;
    }
    if (h.device != c->device) {
      int can = 0;
      DGN_CUDA(cudaDeviceCanAccessPeer(&can, c->device, h.device));
      if (!can) return fail(DGN_ERR_PEER, "device %d cannot access device %d of rank %d", c->device, h.device, j);
    }
    if (h.pid == me_pid) {
      if (h.device != c->device) {
        cudaError_t e = cudaDeviceEnablePeerAccess(h.device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
          return fail(DGN_ERR_PEER, "cudaDeviceEnablePeerAccess(%d): %s", h.device, cudaGetErrorString(e));
        cudaGetLastError();
      }
      c->peer_base[j] = (void*)(uintptr_t)h.base_ptr;
      c->peer_ipc[j] = false;
    } else {
      void* p = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&p, h.ipc, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(DGN_ERR_PEER, "cudaIpcOpenMemHandle for rank %d: %s", j, cudaGetErrorString(e));
      }
      c->peer_base[j] = p;
      c->peer_ipc[j] = true;
    }
  }
  setup_nvls(c, all_handles);
  fill_peer_table(c, &c->table);
  c->connected = true;
  return DGN_OK;
}

int dgn_comm_create(int rank, int nranks, int device, const char* rendezvous_dir, const char* tag,
                    int timeout_ms, dgn_comm_t* comm) {
  if (!comm) return fail(DGN_ERR_ARG, "comm is null");
  *comm = nullptr;
  if (nranks > 1 && (!rendezvous_dir || !tag || !*tag)) return fail(DGN_ERR_ARG, "rendezvous_dir and tag are required");
  dgn_comm* c = nullptr;
  int rc = dgn_comm_init_local(rank, nranks, device, &c);
  if (rc != DGN_OK) return rc;
  if (nranks == 1) {
    *comm = c;
    return DGN_OK;
  }
  std::string dir(rendezvous_dir);
  mkdir(dir.c_str(), 0777);
  auto name = [&](int r, const char* suffix) {
    return dir + "/" + tag + "." + std::to_string(r) + suffix;
  };
  auto drop_mine = [&]() {
    unlink(name(rank, ".h").c_str());
    unlink(name(rank, ".ok").c_str());
  };
  // A run that crashed may have left files under this tag: remove this rank's
  // own before writing.  A peer's stale handle is recognised by its writer
  // being gone; a stale ".ok" by a session number that is not this run's.
  drop_mine();
  char mine[DGN_HANDLE_BYTES];
  rc = dgn_comm_get_handle(c, mine);
  if (rc != DGN_OK) {
    free_comm(c);
    return rc;
  }
  if (!write_file_atomic(name(rank, ".h"), mine, sizeof(mine))) {
    free_comm(c);
    return fail(DGN_ERR_ARG, "cannot write rendezvous file in %s: %s", rendezvous_dir, strerror(errno));
  }
  std::vector<char> all((size_t)nranks * DGN_HANDLE_BYTES);
  const double deadline = now_s() + 1e-3 * (timeout_ms > 0 ? timeout_ms : 60000);
  for (int r = 0; r < nranks; ++r) {
    char* slot = all.data() + (size_t)r * DGN_HANDLE_BYTES;
    for (;;) {
      if (read_file_exact(name(r, ".h"), slot, DGN_HANDLE_BYTES)) {
        Handle h;
        memcpy(&h, slot, sizeof(h));
        // kill(pid, 0): does the writer still exist?  (EPERM means it does.)
        if (h.magic == kMagic && (r == rank || kill((pid_t)h.pid, 0) == 0 || errno == EPERM)) break;
      }
      if (now_s() > deadline) {
        drop_mine();
        free_comm(c);
        return fail(DGN_ERR_TIMEOUT, "rank %d never arrived at rendezvous '%s'", r, tag);
      }
      usleep(500);
    }
  }
  rc = dgn_comm_connect(c, all.data());
  if (rc != DGN_OK) {
    drop_mine();
    free_comm(c);
    return rc;
  }
  // Second phase: nobody removes its handle file before everyone has read it.
  // Each ".ok" carries the session number of rank 0's handle as its writer saw it.
  Handle h0;
  memcpy(&h0, all.data(), sizeof(h0));
  const uint64_t session = h0.session;
  write_file_atomic(name(rank, ".ok"), &session, sizeof(session));
  for (int r = 0; r < nranks; ++r) {
    uint64_t seen = 0;
    while (!read_file_exact(name(r, ".ok"), &seen, sizeof(seen)) || seen != session) {
      if (now_s() > deadline) {
        drop_mine();
        free_comm(c);
        return fail(DGN_ERR_TIMEOUT, "rank %d never finished rendezvous '%s'", r, tag);
      }
      usleep(500);
    }
  }
  unlink(name(rank, ".h").c_str());
  c->rdv_ok_file = name(rank, ".ok");
  *comm = c;
  return DGN_OK;
}

int dgn_comm_create_emulated(int nranks, int device, dgn_comm_t* comms) {
  if (!comms) return fail(DGN_ERR_ARG, "comms is null");
  if (nranks < 1 || nranks > DGN_MAX_RANKS) return fail(DGN_ERR_ARG, "nranks %d outside 1..%d", nranks, DGN_MAX_RANKS);
  Team* t = new Team();
  t->n = nranks;
  t->device = device;
  for (int r = 0; r < nranks; ++r) {
    dgn_comm* c = nullptr;
    g_skip_nvls = true;
    int rc = dgn_comm_init_local(r, nranks, device, &c);
    g_skip_nvls = false;
    if (rc != DGN_OK) {
      for (dgn_comm* m : t->members) free_comm(m);
      delete t;
      return rc;
    }
    c->team = t;
    t->members.push_back(c);
  }
  for (int r = 0; r < nranks; ++r) {
    dgn_comm* c = t->members[r];
    for (int j = 0; j < nranks; ++j) c->peer_base[j] = t->members[j]->base;
    fill_peer_table(c, &c->table);
  }
  t->alive = nranks;
  for (int r = 0; r < nranks; ++r) {
    t->members[r]->connected = true;
    comms[r] = t->members[r];
  }
  return DGN_OK;
}

int dgn_comm_destroy(dgn_comm_t c) {
  if (!c) return DGN_OK;
  Team* t = c->team;
  if (t) {
    for (auto& m : t->members)
      if (m == c) m = nullptr;
    if (--t->alive == 0) delete t;
  }
  free_comm(c);
  return DGN_OK;
}

int dgn_comm_rank(dgn_comm_t c) { return c ? c->rank : -1; }
int dgn_comm_size(dgn_comm_t c) { return c ? c->nranks : 0; }
int dgn_comm_device(dgn_comm_t c) { return c ? c->device : -1; }
int dgn_comm_status(dgn_comm_t c) { return (c && c->status_host) ? *(volatile int*)c->status_host : DGN_ERR_ARG; }

int dgn_comm_set_wait_limit_ms(dgn_comm_t c, int ms) {
  if (!c || ms < 1) return fail(DGN_ERR_ARG, "bad wait limit");
  c->wait_ns = (u64)ms * 1000000ull;
  return DGN_OK;
}

int dgn_comm_set_tuning(dgn_comm_t c, int variant, int blocks, int threads, int64_t chunk_bytes) {
  if (!c) return fail(DGN_ERR_ARG, "null communicator");
  if (variant < 0 || variant > DGN_VARIANT_RING_PULL || blocks < 0 || threads < 0 || chunk_bytes < 0)
    return fail(DGN_ERR_ARG, "bad tuning value");
  if ((variant == DGN_VARIANT_NVLS || variant == DGN_VARIANT_SYMM) && !c->nvls)
    return fail(DGN_ERR_UNSUPPORTED, "the NVLS variants are not set up on this communicator");
  c->tune_variant = variant;
  c->tune_blocks = blocks;
  c->tune_threads = threads;
  c->tune_chunk = chunk_bytes;
  return DGN_OK;
}

int dgn_comm_set_knob(dgn_comm_t c, const char* name, int64_t value) {
  if (!c || !name) return fail(DGN_ERR_ARG, "null argument");
  if (value < 0) return fail(DGN_ERR_ARG, "knob %s: negative value", name);
  const std::string k(name);
  if (k == "flow_chunk_bytes") c->flow_chunk_bytes = value;
  else if (k == "flow_switch_blocks") c->flow_switch_blocks = (int)value;
  else if (k == "flow_in_blocks") c->flow_in_blocks = (int)value;
  else if (k == "flow_out_blocks") c->flow_out_blocks = (int)value;
  else if (k == "flow_depth") c->flow_depth = (int)value;
  else if (k == "nvls_unroll") c->unroll = (int)value;
  else if (k == "nvls_pattern") c->pattern = (int)value;
  else if (k == "nvls_min_bytes") c->nvls_min_bytes = value;
  else if (k == "symm_min_bytes") c->symm_min_bytes = value;
  else if (k == "nvls_bcast_min_bytes") c->nvls_bcast_min_bytes = value;
  else if (k == "bcast_scatter_min_bytes") c->bcast_scatter_min_bytes = value;
  else if (k == "allgather_pull_min_bytes") c->allgather_pull_min_bytes = value;
  else if (k == "nvls_allgather_min_bytes") c->nvls_allgather_min_bytes = value;
  else if (k == "gather_chunk_bytes") c->gather_chunk_bytes = value;
  else if (k == "gather_push_blocks") c->gather_push_blocks = (int)value;
  else if (k == "gather_forward_blocks") c->gather_forward_blocks = (int)value;
  else if (k == "gather_mode") c->gather_mode = (int)value;
  else if (k == "bcast_shard_min_bytes") c->bcast_shard_min_bytes = value;
  else if (k == "allgather_ring_min_bytes") c->allgather_ring_min_bytes = value;
  else return fail(DGN_ERR_ARG, "unknown knob '%s'", name);
  return DGN_OK;
}

int dgn_comm_has_nvls(dgn_comm_t c) { return (c && c->nvls) ? 1 : 0; }

int dgn_allreduce(dgn_comm_t c, const void* const* in_ptrs, void* const* out_ptrs,
                  const int64_t* counts, int ntensors, int dtype, int redop, void* stream) {
  int rc = check_ready(c);
  if (rc != DGN_OK) return rc;
  if (ntensors < 0 || (ntensors > 0 && (!in_ptrs || !out_ptrs || !counts)))
    return fail(DGN_ERR_ARG, "null tensor list");
  const size_t es = dgn_dtype_size(dtype);
  if (es == 0) return fail(DGN_ERR_ARG, "unknown dtype %d", dtype);
  if (redop < DGN_SUM || redop > DGN_MAX) return fail(DGN_ERR_ARG, "unknown reduction %d", redop);
  if (redop == DGN_MEAN && dtype <= DGN_I64)
    return fail(DGN_ERR_UNSUPPORTED, "MEAN is defined for floating-point types only");
  long long total = 0;
  for (int i = 0; i < ntensors; ++i) {
    if (counts[i] < 0) return fail(DGN_ERR_ARG, "negative count for tensor %d", i);
    if (counts[i] > 0 && (!in_ptrs[i] || !out_ptrs[i])) return fail(DGN_ERR_ARG, "null pointer for tensor %d", i);
    total += counts[i];
  }
  if (total == 0) return DGN_OK;
  if (ntensors > kMaxTableTensors) {  // more entries than one launch takes
    for (int i = 0; i < ntensors; i += kMaxTableTensors) {
      const int m = ntensors - i < kMaxTableTensors ? ntensors - i : kMaxTableTensors;
      rc = dgn_allreduce(c, in_ptrs + i, out_ptrs + i, counts + i, m, dtype, redop, stream);
      if (rc != DGN_OK) return rc;
    }
    return DGN_OK;
  }
  OpDesc d;
  d.kind = kOpAllReduce;
  d.dtype = dtype;
  d.redop = redop;
  d.stream = static_cast<cudaStream_t>(stream);
  // A list with a single non-empty tensor is the flat case.
  int nonempty = 0, only = -1;
  for (int i = 0; i < ntensors; ++i)
    if (counts[i] > 0) { ++nonempty; only = i; }
  if (nonempty == 1) {
    d.ntensors = 1;
    d.count = counts[only];
    d.nvec = ceil_div(d.count * (long long)es, 16);
    d.in = in_ptrs[only];
    d.out = out_ptrs[only];
  } else {
    DeviceGuard g(c->device);
    const TableEntry* te = nullptr;
    rc = get_table(c, in_ptrs, out_ptrs, counts, ntensors, (int)es, d.stream, &te);
    if (rc != DGN_OK) return rc;
    d.ntensors = te->nt;
    d.count = total;
    d.nvec = te->nvec;
    d.table = te->d_table;
    if (d.nvec >= (1ll << 32)) return fail(DGN_ERR_UNSUPPORTED, "bucket larger than 64 GiB");
  }
  if (c->nranks == 1) {
    bool inplace = true;
    for (int i = 0; i < ntensors; ++i)
      if (counts[i] > 0 && in_ptrs[i] != out_ptrs[i]) inplace = false;
    if (inplace) return DGN_OK;  // nothing to move, as in collective_op.cc:89
    return launch_local_copy(c, d, (int)es);
  }
  return issue(c, d);
}

int dgn_allreduce_host(dgn_comm_t c, const void* in, void* out, int64_t count, int dtype, int redop) {
  int rc = check_ready(c);
  if (rc != DGN_OK) return rc;
  if (c->team) return fail(DGN_ERR_UNSUPPORTED, "the host all-reduce blocks and cannot run on an emulated communicator");
  const size_t es = dgn_dtype_size(dtype);
  if (es == 0) return fail(DGN_ERR_ARG, "unknown dtype %d", dtype);
  if (count < 0) return fail(DGN_ERR_ARG, "negative count");
  if (count == 0) return DGN_OK;
  if (!in || !out) return fail(DGN_ERR_ARG, "null pointer");
  const size_t bytes = (size_t)count * es;
  if (bytes > 4096) return fail(DGN_ERR_ARG, "the host all-reduce takes at most 4096 bytes, got %zu", bytes);
  if (c->nranks == 1) {
    if (in != out) memmove(out, in, bytes);
    return DGN_OK;
  }
  DeviceGuard g(c->device);
  // Kernels of one communicator must not overlap: wait for the latest one.
  if (c->has_last_stream) DGN_CUDA(cudaStreamSynchronize(c->last_stream));
  memcpy(c->host_pin, in, bytes);
  DGN_CUDA(cudaMemcpyAsync(c->host_dev, c->host_pin, bytes, cudaMemcpyHostToDevice, c->host_stream));
  const void* ins[1] = {c->host_dev};
  void* outs[1] = {c->host_dev};
  int64_t counts[1] = {count};
  rc = dgn_allreduce(c, ins, outs, counts, 1, dtype, redop, c->host_stream);
  if (rc != DGN_OK) return rc;
  DGN_CUDA(cudaMemcpyAsync(c->host_pin, c->host_dev, bytes, cudaMemcpyDeviceToHost, c->host_stream));
  DGN_CUDA(cudaStreamSynchronize(c->host_stream));
  if (dgn_comm_status(c) != DGN_OK) return fail(DGN_ERR_TIMEOUT, "a peer did not join the host all-reduce in time");
  memcpy(out, c->host_pin, bytes);
  return DGN_OK;
}

int dgn_reducescatter(dgn_comm_t c, const void* in, void* out, int64_t count, int dtype, int redop,
                      void* stream) {
  int rc = check_ready(c);
  if (rc != DGN_OK) return rc;
  const size_t es = dgn_dtype_size(dtype);
  if (es == 0) return fail(DGN_ERR_ARG, "unknown dtype %d", dtype);
  if (redop < DGN_SUM || redop > DGN_MAX) return fail(DGN_ERR_ARG, "unknown reduction %d", redop);
  if (redop == DGN_MEAN && dtype <= DGN_I64)
    return fail(DGN_ERR_UNSUPPORTED, "MEAN is defined for floating-point types only");
  if (count < 0) return fail(DGN_ERR_ARG, "negative count");
  if (count == 0) return DGN_OK;
  if (!in || !out) return fail(DGN_ERR_ARG, "null pointer");
  OpDesc d;
  d.kind = kOpReduceScatter;
  d.dtype = dtype;
  d.redop = redop;
  d.count = count;
  d.nvec = ceil_div(count * (long long)es, 16);
  d.in = in;
  d.out = out;
  d.stream = static_cast<cudaStream_t>(stream);
  if (c->nranks == 1) {
    if (in == out) return DGN_OK;
    return launch_local_copy(c, d, (int)es);
  }
  return issue(c, d);
}

int dgn_allgather(dgn_comm_t c, const void* in, void* out, int64_t count, int dtype, void* stream) {
  int rc = check_ready(c);
  if (rc != DGN_OK) return rc;
  const size_t es = dgn_dtype_size(dtype);
  if (es == 0) return fail(DGN_ERR_ARG, "unknown dtype %d", dtype);
  if (count < 0) return fail(DGN_ERR_ARG, "negative count");
  if (count == 0) return DGN_OK;
  if (!in || !out) return fail(DGN_ERR_ARG, "null pointer");
  OpDesc d;
  d.kind = kOpAllGather;
  d.dtype = DGN_U8;
  d.count = count * (long long)es;  // bytes per rank
  d.nvec = ceil_div(d.count, 16);
  d.in = in;
  d.out = out;
  d.stream = static_cast<cudaStream_t>(stream);
  if (c->nranks == 1) {
    if (in == out) return DGN_OK;
    return launch_local_copy(c, d, 1);
  }
  return issue(c, d);
}

int dgn_broadcast(dgn_comm_t c, void* buf, int64_t count, int dtype, int root, void* stream) {
  int rc = check_ready(c);
  if (rc != DGN_OK) return rc;
  const size_t es = dgn_dtype_size(dtype);
  if (es == 0) return fail(DGN_ERR_ARG, "unknown dtype %d", dtype);
  if (count < 0) return fail(DGN_ERR_ARG, "negative count");
  if (root < 0 || root >= c->nranks) return fail(DGN_ERR_ARG, "root %d outside 0..%d", root, c->nranks - 1);
  if (count == 0 || c->nranks == 1) return DGN_OK;
  if (!buf) return fail(DGN_ERR_ARG, "null pointer");
  OpDesc d;
  d.kind = kOpBroadcast;
  d.dtype = DGN_U8;
  d.root = root;
  d.count = count * (long long)es;
  d.nvec = ceil_div(d.count, 16);
  d.in = buf;
  d.out = buf;
  d.stream = static_cast<cudaStream_t>(stream);
  return issue(c, d);
}

int64_t dgn_zero_shard_count(int nranks, int64_t total) {
  if (nranks < 1 || total < 0) return -1;
  return ceil_div(total, nranks);
}

int64_t dgn_zero_state_count(int nranks, int64_t total, int dtype) {
  const size_t es = dgn_dtype_size(dtype);
  if (nranks < 1 || total < 0 || es == 0) return -1;
  const long long E = 16 / (long long)es;
  return (ceil_div(ceil_div(total, nranks), E) + 1) * E;
}

int64_t dgn_zero_state_offset(int rank, int nranks, int64_t total, int dtype) {
  const size_t es = dgn_dtype_size(dtype);
  if (nranks < 1 || rank < 0 || rank >= nranks || total < 0 || es == 0) return -1;
  const ShardGeom sg = shard_geom(total, ceil_div(total, nranks), rank, (int)(16 / es));
  return sg.e_lo - sg.g_lo * (long long)(16 / es);
}

int dgn_zero_init_master(dgn_comm_t c, const void* const* param_ptrs, const int64_t* counts, int ntensors,
                         int dtype, float* master, void* stream) {
  int rc = check_ready(c);
  if (rc != DGN_OK) return rc;
  long long total = 0;
  int nonempty = 0;
  rc = check_zero_bucket(param_ptrs, param_ptrs, counts, ntensors, dtype, &total, &nonempty);
  if (rc != DGN_OK) return rc;
  if (total == 0) return DGN_OK;
  if (!master || ((uintptr_t)master & 15u)) return fail(DGN_ERR_ARG, "master must be a 16-byte aligned device pointer");
  if (c->team && !c->team->pending[c->rank].empty())
    return fail(DGN_ERR_STATE, "virtual rank %d still has collectives waiting for the other ranks", c->rank);
  DeviceGuard g(c->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const ZeroTableEntry* te = nullptr;
  rc = get_zero_table(c, param_ptrs, const_cast<void* const*>(param_ptrs), counts, ntensors, nullptr,
                      (int)kElemSize[dtype], s, &te);
  if (rc != DGN_OK) return rc;
  OpDesc d;
  d.kind = kOpZeroReduce;
  d.dtype = dtype;
  d.count = total;
  d.ntensors = te->nt;
  d.stream = s;
  Plan p;
  ZeroParams Z;
  fill_zero_params(&Z, c, d, p);
  Z.base.peers[0] = c->table;
  Z.zr[0].table = te->d_table;
  Z.zr[0].master = master;
  const long long E = 16 / (long long)kElemSize[dtype];
  const long long nv = ceil_div(ceil_div(total, c->nranks), E) + 1;
  long long blocks = ceil_div(nv, 256);
  if (blocks > (long long)c->num_sms * 8) blocks = (long long)c->num_sms * 8;
  return launch(zero_kernel_fn(dtype, 2), dim3((unsigned)blocks, 1), 256, zero_smem_bytes(te->nt), s, &Z, false);
}

int dgn_zero_adamw(dgn_comm_t c, const void* const* grad_ptrs, void* const* param_ptrs, const int64_t* counts,
                   int ntensors, int dtype, float* master, float* m, float* v, float* grad_shard,
                   const float* lr_scales, const dgn_adamw_args* args, float* found_inf, void* stream) {
  int rc = check_ready(c);
  if (rc != DGN_OK) return rc;
  if (!args) return fail(DGN_ERR_ARG, "null hyper-parameters");
  long long total = 0;
  int nonempty = 0;
  rc = check_zero_bucket(grad_ptrs, const_cast<const void* const*>(param_ptrs), counts, ntensors, dtype, &total,
                         &nonempty);
  if (rc != DGN_OK) return rc;
  if (total == 0) return DGN_OK;
  if (!master || !m || !v || !grad_shard)
    return fail(DGN_ERR_ARG, "master, m, v and grad_shard are required");
  if (((uintptr_t)master | (uintptr_t)m | (uintptr_t)v | (uintptr_t)grad_shard) & 15u)
    return fail(DGN_ERR_ARG, "master, m, v and grad_shard must be 16-byte aligned");
  DeviceGuard g(c->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bool scaled = false;
  if (lr_scales)
    for (int i = 0; i < ntensors; ++i) scaled = scaled || lr_scales[i] != 1.f;
  const ZeroTableEntry* te = nullptr;
  rc = get_zero_table(c, grad_ptrs, param_ptrs, counts, ntensors, scaled ? lr_scales : nullptr,
                      (int)kElemSize[dtype], s, &te);
  if (rc != DGN_OK) return rc;
  OpDesc d;
  d.kind = kOpZeroReduce;
  d.dtype = dtype;
  d.count = total;
  d.nvec = ceil_div(total * (long long)kElemSize[dtype], 16);
  d.ntensors = te->nt;
  d.stream = s;
  d.zr.table = te->d_table;
  d.zr.master = master;
  d.zr.m = m;
  d.zr.v = v;
  d.zr.gshard = grad_shard;
  d.zr.found_inf = found_inf;
  d.zh.lr = args->lr;
  d.zh.beta1 = args->beta1;
  d.zh.beta2 = args->beta2;
  d.zh.eps = args->eps;
  d.zh.wd = args->weight_decay;
  d.zh.grad_scale = args->grad_scale;
  d.zh.clip_norm = args->clip_norm;
  d.zh.clip_value = args->clip_value;
  d.zh.check_finite = found_inf ? 1 : 0;
  d.zh.use_lr_scales = scaled ? 1 : 0;
  rc = issue(c, d);
  if (rc != DGN_OK) return rc;
  d.kind = kOpZeroUpdate;
  return issue(c, d);
}

int dgn_allreduce_update(dgn_comm_t c, const void* const* grad_ptrs, void* const* param_ptrs, void* const* m_ptrs,
                         void* const* v_ptrs, const int64_t* counts, int ntensors, int dtype,
                         const dgn_update_args* args, void* stream) {
  int rc = check_ready(c);
  if (rc != DGN_OK) return rc;
  if (!args) return fail(DGN_ERR_ARG, "null hyper-parameters");
  if (dtype != DGN_F32) return fail(DGN_ERR_UNSUPPORTED, "the fused update takes float32 tensors, got dtype %d", dtype);
  if (args->kind < DGN_UPDATE_MOMENTUM_SGD || args->kind > DGN_UPDATE_ADAMW)
    return fail(DGN_ERR_ARG, "unknown update kind %d", args->kind);
  const bool two = args->kind == DGN_UPDATE_ADAM || args->kind == DGN_UPDATE_ADAMW;
  if (ntensors < 1 || !grad_ptrs || !param_ptrs || !m_ptrs || !counts || (two && !v_ptrs))
    return fail(DGN_ERR_ARG, "null or empty tensor list");
  long long total = 0;
  int nonempty = 0;
  for (int i = 0; i < ntensors; ++i) {
    if (counts[i] < 0) return fail(DGN_ERR_ARG, "negative count for tensor %d", i);
    if (counts[i] == 0) continue;
    if (!grad_ptrs[i] || !param_ptrs[i] || !m_ptrs[i] || (two && !v_ptrs[i]))
      return fail(DGN_ERR_ARG, "null pointer for tensor %d", i);
    if (((uintptr_t)grad_ptrs[i] | (uintptr_t)param_ptrs[i] | (uintptr_t)m_ptrs[i] | (two ? (uintptr_t)v_ptrs[i] : 0)) & 3u)
      return fail(DGN_ERR_ARG, "tensor %d is not aligned to its element size", i);
    total += counts[i];
    ++nonempty;
  }
  if (total == 0) return DGN_OK;
  if (nonempty > 512) return fail(DGN_ERR_UNSUPPORTED, "a fused update takes at most 512 tensors per call, got %d", nonempty);
  DeviceGuard g(c->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const UpdTableEntry* te = nullptr;
  rc = get_update_table(c, grad_ptrs, param_ptrs, m_ptrs, two ? v_ptrs : nullptr, counts, ntensors, s, &te);
  if (rc != DGN_OK) return rc;
  if (te->nvec >= (1ll << 32)) return fail(DGN_ERR_UNSUPPORTED, "bucket larger than 64 GiB");
  OpDesc d;
  d.kind = kOpAllReduceUpdate;
  d.dtype = DGN_F32;
  d.redop = DGN_SUM;
  d.count = total;
  d.nvec = te->nvec;
  d.ntensors = te->nt;
  d.stream = s;
  d.utable = te->d_table;
  d.uh.kind = args->kind;
  d.uh.lr = args->lr;
  d.uh.a = two ? args->beta1 : args->momentum;
  d.uh.b = args->beta2;
  d.uh.eps = args->eps;
  d.uh.wd = args->weight_decay;
  d.uh.grad_scale = args->grad_scale;
  d.uh.clip_value = args->clip_value;
  return issue(c, d);
}

int dgn_plan_query(int nranks, int num_sms, int has_nvls, int64_t symm_bytes, int in_symm, int op, int dtype,
                   int redop, int64_t count, int ntensors, int* variant, int* blocks, int* threads,
                   int64_t* chunk_bytes, int* rounds) {
  if (nranks < 2 || nranks > DGN_MAX_RANKS) return fail(DGN_ERR_ARG, "nranks %d outside 2..%d", nranks, DGN_MAX_RANKS);
  const size_t es = dgn_dtype_size(dtype);
  if (es == 0 || count <= 0 || num_sms < 1 || ntensors < 1 || op < kOpAllReduce || op > kOpBroadcast)
    return fail(DGN_ERR_ARG, "bad plan query");
  dgn_comm q;
  q.nranks = nranks;
  q.num_sms = num_sms;
  load_thresholds(&q);
  if (has_nvls) {
    load_nvls_settings(&q, symm_bytes);
    q.nvls = reinterpret_cast<NvlsBuffer*>(&q);  // only its presence is looked at
  }
  q.plan_query = true;
  q.plan_query_in_symm = in_symm != 0;
  OpDesc d;
  d.kind = op;
  d.dtype = (op == kOpAllGather || op == kOpBroadcast) ? (int)DGN_U8 : dtype;
  d.redop = redop;
  d.ntensors = ntensors;
  d.count = (op == kOpAllGather || op == kOpBroadcast) ? count * (long long)es : count;
  d.nvec = ceil_div(count * (long long)es, 16);
  d.in = d.out = reinterpret_cast<void*>(16);  // in place
  const Plan p = make_plan(&q, d, 0);
  q.nvls = nullptr;
  if (variant) *variant = p.variant;
  if (blocks) *blocks = p.blocks;
  if (threads) *threads = p.threads;
  if (chunk_bytes) *chunk_bytes = (int64_t)p.cv * 16;
  if (rounds) *rounds = p.rounds;
  return DGN_OK;
}

int dgn_plan_query_staged(int nranks, int num_sms, int has_nvls, int op, int64_t bytes, dgn_staged_plan* out) {
  if (!out) return fail(DGN_ERR_ARG, "null argument");
  if (nranks < 2 || nranks > DGN_MAX_RANKS) return fail(DGN_ERR_ARG, "nranks %d outside 2..%d", nranks, DGN_MAX_RANKS);
  if (bytes <= 0 || num_sms < 1 || (op != kOpAllReduce && op != kOpAllGather && op != kOpBroadcast))
    return fail(DGN_ERR_ARG, "bad plan query");
  dgn_comm q;
  q.nranks = nranks;
  q.num_sms = num_sms;
  load_thresholds(&q);
  if (has_nvls) {
    load_nvls_settings(&q, 0);
    q.nvls = reinterpret_cast<NvlsBuffer*>(&q);  // only its presence is looked at
  }
  q.plan_query = true;
  OpDesc d;
  d.kind = op;
  d.dtype = op == kOpAllReduce ? (int)DGN_F32 : (int)DGN_U8;
  d.redop = DGN_SUM;
  d.ntensors = 1;
  d.count = op == kOpAllReduce ? bytes / 4 : bytes;
  d.nvec = ceil_div(bytes, 16);
  d.in = d.out = reinterpret_cast<void*>(16);
  const Plan p = make_plan(&q, d, 0);
  q.nvls = nullptr;
  memset(out, 0, sizeof(*out));
  out->variant = p.variant;
  out->blocks = p.blocks;
  out->threads = p.threads;
  out->chunks = p.rounds;
  out->chunk_vectors = p.cv;
  const bool staged = p.variant == DGN_VARIANT_NVLS || p.variant == DGN_VARIANT_RING || p.variant == DGN_VARIANT_RING_PULL;
  if (!staged) return DGN_OK;
  out->staged = 1;
  out->depth = p.flow_depth;
  out->first_role_blocks = p.flow_nsw;
  out->second_role_blocks = p.flow_nin;
  const long long half = (long long)q.geo.ring_bytes / 2;
  const bool through_switch = p.variant == DGN_VARIANT_NVLS;
  if (op == kOpAllReduce) {
    out->ring_bytes_needed = (int64_t)p.flow_depth * p.cv * 16;
    out->ring_bytes_available = through_switch ? (int64_t)q.flow_ring_bytes : half;
  } else {
    const bool scatter = (p.flow_mode & kGatherScatter) != 0, pull = (p.flow_mode & kGatherPull) != 0;
    const int regions = pull ? 1 : (op == kOpAllGather || scatter) ? nranks : 1;
    out->mode = p.flow_mode;
    out->ring_bytes_needed = (int64_t)p.flow_depth * regions * p.cv * 16;
    out->ring_bytes_available = through_switch ? (int64_t)q.gather_ring_bytes : half;
    if (scatter) {
      out->inbox_bytes_needed = (int64_t)p.flow_depth * p.cv * 16;
      // Through the switch the inboxes have the gather half of the workspace ring to
      // themselves; otherwise they lie behind the ring inside that half.
      out->inbox_offset_in_half = p.inbox_off - ((int64_t)q.geo.ring_off + half);
      out->inbox_bytes_available = half - out->inbox_offset_in_half;
    }
  }
  return DGN_OK;
}

int64_t dgn_launch_count(void) { return g_launches.load(); }

int dgn_comm_last_launch(dgn_comm_t c, int* variant, int* blocks, int* threads, int64_t* chunk_bytes,
                         int* rounds) {
  if (!c) return fail(DGN_ERR_ARG, "null communicator");
  if (variant) *variant = c->last_plan.variant;
  if (blocks) *blocks = c->last_plan.blocks;
  if (threads) *threads = c->last_plan.threads;
  if (chunk_bytes) *chunk_bytes = (int64_t)c->last_plan.cv * 16;
  if (rounds) *rounds = c->last_plan.rounds;
  return DGN_OK;
}

}  // extern "C"
