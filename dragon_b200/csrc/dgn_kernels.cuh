// Device side of the B200-native `Collective` path: peer-memory kernels for
// ALLREDUCE (one-shot and two-shot), REDUCESCATTER, ALLGATHER, BROADCAST and
// the single-rank copy path.
//
// Memory model.  Every rank owns one "symmetric workspace" that all peers map
// (CUDA IPC across processes, peer access inside one process):
//
//   flags   u64[max_blocks][kMaxRanks]   slot [b][s] is written only by block b
//                                        of rank s, with strictly increasing
//                                        epoch numbers (never reset)
//   stage   for parity p in {0,1}, block b: (nranks + 1) slots of slot_bytes
//           slot s < nranks : "inbox" written by rank s (peer stores)
//           slot nranks     : "outbox" written by the owner, read by peers
//
// Block b of one rank only ever talks to block b of the other ranks, so a
// collective needs no grid-wide barrier: each block runs
//   pre-wait -> (push | publish) -> signal -> wait -> reduce/pull -> ... -> done
// on its own slice of the message.  All waits are bounded: when the limit runs
// out the block records DGN_ERR_TIMEOUT in the status word and leaves.
//
// Protocol state is device-resident: block b keeps its next epoch number, its
// collective count (whose low bit is the staging parity) and, per parity, the
// epoch with which it last finished, in its own BlockState.  Every rank runs
// the same sequence of collectives with the same launch shapes, so block b of
// every rank holds the same numbers without any host bookkeeping, and a
// captured launch can be replayed.
//
// Reuse safety.  Consecutive collectives of a block alternate parity.  Before
// a block touches any peer's parity-p region again it waits until every
// peer's block b has signalled the epoch with which the previous parity-p
// collective finished ("done" signal), i.e. has stopped reading its data.
//
// Data always moves as 16-byte vectors with ld/st.global.cg (L2-coherent, no
// L1 allocation), so data published by a peer before its release-store of a
// flag is seen after the acquire-load of that flag.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dgn {

constexpr int kMaxRanks = 8;
constexpr int kMaxTableTensors = 1024;  // bucket entries one launch can take

enum : int { kU8 = 0, kI8, kI32, kI64, kF16, kBF16, kF32, kF64 };
enum : int { kSum = 0, kMean, kProd, kMin, kMax };
enum : int { kErrTimeout = 3 };

typedef unsigned long long u64;

// Per-block protocol state (local device memory, touched by block b only).
struct BlockState {
  u64 epoch;         // last epoch number used by this block
  u64 ops;           // collectives this block took part in; low bit = parity
  u64 last_done[2];  // per parity: epoch of the last "done" signal
};

// One rank's view of the team.  Lives in that rank's device memory.
struct PeerTable {
  char* stage[kMaxRanks];  // rank j's staging base, as mapped on this device
  u64* flags[kMaxRanks];   // rank j's flag array, as mapped on this device
  struct BlockState* blk;  // [max_blocks], local
  int* status;             // error word (pinned host memory, device-visible)
  int rank, nranks, max_blocks, reserved;
  long long slot_bytes;    // bytes per slot
};

// One tensor of a bucket; `vbegin` is its first 16-byte vector in the flat
// message (each tensor starts on a vector boundary of the flat message).
struct TensorEnt {
  const char* in;
  char* out;
  long long count;   // elements
  long long vbegin;  // flat vector index
};

struct RankArgs {
  const void* in;
  void* out;
  const TensorEnt* table;  // device memory, ntensors (+1 sentinel) entries
};

struct OpParams {
  const PeerTable* peers;  // [gridDim.y]
  RankArgs ra[kMaxRanks];  // indexed by blockIdx.y
  long long count;         // elements per rank (single tensor / per-rank block)
  long long nvec;          // flat 16-byte vectors of the message
  u64 wait_ns;
  double scale;            // MEAN factor, double(1.f / float(nranks))
  int ntensors;
  int rounds;
  int cv;                  // vectors per block per round (<= slot_bytes / 16)
  int redop;
  int root;
};

// ---------------------------------------------------------------------------
// flags

__device__ __forceinline__ void st_release_sys(u64* p, u64 v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u64 ld_acquire_sys(const u64* p) {
  u64 v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ u64 global_timer_ns() {
  u64 t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Publishes everything this block has stored so far, then tells block `b` of
// the peers (all, or only `only`) that epoch `val` is reached.
__device__ __forceinline__ void signal_peers(const PeerTable& pt, int b, u64 val, int only = -1) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < pt.nranks && t != pt.rank && (only < 0 || t == only))
    st_release_sys(pt.flags[t] + (size_t)b * kMaxRanks + pt.rank, val);
}

// Waits until block `b` of the peers (all, or only `only`) has reached epoch
// `target`.  Returns false, for the whole block, if the limit ran out.
__device__ __forceinline__ bool wait_peers(const PeerTable& pt, int b, u64 target, u64 wait_ns,
                                           int only = -1) {
  bool ok = true;
  const int t = threadIdx.x;
  if (t < pt.nranks && t != pt.rank && (only < 0 || t == only)) {
    const u64* f = pt.flags[pt.rank] + (size_t)b * kMaxRanks + t;
    if (ld_acquire_sys(f) < target) {
      const u64 t0 = global_timer_ns();
      unsigned spins = 0;
      for (;;) {
        if (ld_acquire_sys(f) >= target) break;
        if ((++spins & 31u) == 0u && global_timer_ns() - t0 > wait_ns) {
          *(volatile int*)pt.status = kErrTimeout;
          ok = false;
          break;
        }
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

// ---------------------------------------------------------------------------
// 16-byte vector access

__device__ __forceinline__ uint4 ldv(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void stv(void* p, uint4 v) { __stcg(reinterpret_cast<uint4*>(p), v); }

template <int ES> struct Bits;
template <> struct Bits<1> { typedef unsigned char type; };
template <> struct Bits<2> { typedef unsigned short type; };
template <> struct Bits<4> { typedef unsigned int type; };
template <> struct Bits<8> { typedef unsigned long long type; };

// Vector `lv` of a tensor of `count` elements of ES bytes at `base`.  Full,
// 16-byte aligned vectors take one load; a ragged tail or an unaligned base
// is assembled element by element (missing elements read as zero).
template <int ES>
__device__ __forceinline__ uint4 load_vec(const char* base, long long lv, long long count,
                                          bool aligned) {
  constexpr int E = 16 / ES;
  const long long e0 = lv * E;
  if (aligned && e0 + E <= count) return ldv(base + lv * 16);
  typedef typename Bits<ES>::type B;
  union { uint4 v; B e[E]; } u;
  u.v = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int k = 0; k < E; ++k)
    if (e0 + k < count) u.e[k] = __ldcg(reinterpret_cast<const B*>(base) + e0 + k);
  return u.v;
}

template <int ES>
__device__ __forceinline__ void store_vec(char* base, long long lv, long long count, bool aligned,
                                          uint4 x) {
  constexpr int E = 16 / ES;
  const long long e0 = lv * E;
  if (aligned && e0 + E <= count) { stv(base + lv * 16, x); return; }
  typedef typename Bits<ES>::type B;
  union { uint4 v; B e[E]; } u;
  u.v = x;
#pragma unroll
  for (int k = 0; k < E; ++k)
    if (e0 + k < count) __stcg(reinterpret_cast<B*>(base) + e0 + k, u.e[k]);
}

__device__ __forceinline__ bool is_al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The message as a flat sequence of 16-byte vectors.
//  kFlat  : one tensor, vector v = elements [v*E, v*E+E)
//  kTable : a bucket of tensors; shared memory holds the table
template <int ES, bool TABLE>
struct Message {
  const char* in;
  char* out;
  long long count;
  bool in_al, out_al;
  // table mode (arrays in shared memory)
  int nt;
  const unsigned* vbeg;     // [nt + 1]
  const long long* tcount;  // [nt]
  const char* const* tin;   // [nt]
  char* const* tout;        // [nt]

  __device__ __forceinline__ int find(long long v) const {
    int lo = 0, hi = nt;  // invariant: vbeg[lo] <= v < vbeg[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if ((long long)vbeg[mid] <= v) lo = mid; else hi = mid;
    }
    return lo;
  }
  __device__ __forceinline__ uint4 load(long long v) const {
    if (!TABLE) return load_vec<ES>(in, v, count, in_al);
    const int t = find(v);
    const char* p = tin[t];
    return load_vec<ES>(p, v - vbeg[t], tcount[t], is_al16(p));
  }
  __device__ __forceinline__ void store(long long v, uint4 x) const {
    if (!TABLE) { store_vec<ES>(out, v, count, out_al, x); return; }
    const int t = find(v);
    char* p = tout[t];
    store_vec<ES>(p, v - vbeg[t], tcount[t], is_al16(p), x);
  }
};

// Shared-memory footprint of a table of nt tensors.
__host__ __device__ inline size_t table_smem_bytes(int nt) {
  return (size_t)nt * (8 + 8 + 8) + (size_t)(nt + 1) * 4 + 16;
}

template <int ES, bool TABLE>
__device__ __forceinline__ Message<ES, TABLE> make_message(const OpParams& P, const RankArgs& ra,
                                                           unsigned char* smem) {
  Message<ES, TABLE> m;
  m.in = static_cast<const char*>(ra.in);
  m.out = static_cast<char*>(ra.out);
  m.count = P.count;
  m.in_al = is_al16(ra.in);
  m.out_al = is_al16(ra.out);
  m.nt = P.ntensors;
  m.vbeg = nullptr; m.tcount = nullptr; m.tin = nullptr; m.tout = nullptr;
  if (TABLE) {
    const int nt = P.ntensors;
    const char** tin = reinterpret_cast<const char**>(smem);
    char** tout = reinterpret_cast<char**>(smem + (size_t)nt * 8);
    long long* tc = reinterpret_cast<long long*>(smem + (size_t)nt * 16);
    unsigned* vb = reinterpret_cast<unsigned*>(smem + (size_t)nt * 24);
    for (int i = threadIdx.x; i < nt; i += blockDim.x) {
      const TensorEnt e = ra.table[i];
      tin[i] = e.in; tout[i] = e.out; tc[i] = e.count; vb[i] = (unsigned)e.vbegin;
    }
    if (threadIdx.x == 0) vb[nt] = (unsigned)P.nvec;
    __syncthreads();
    m.tin = tin; m.tout = tout; m.tcount = tc; m.vbeg = vb;
  }
  return m;
}

// ---------------------------------------------------------------------------
// reductions

template <typename T> struct Elem;  // E, Acc, unpack, pack
template <> struct Elem<float> {
  static constexpr int E = 4; typedef float Acc;
  static __device__ __forceinline__ void unpack(uint4 v, Acc* a) {
    a[0] = __uint_as_float(v.x); a[1] = __uint_as_float(v.y);
    a[2] = __uint_as_float(v.z); a[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const Acc* a) {
    return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]),
                      __float_as_uint(a[3]));
  }
};
template <> struct Elem<double> {
  static constexpr int E = 2; typedef double Acc;
  static __device__ __forceinline__ void unpack(uint4 v, Acc* a) {
    a[0] = __hiloint2double((int)v.y, (int)v.x); a[1] = __hiloint2double((int)v.w, (int)v.z);
  }
  static __device__ __forceinline__ uint4 pack(const Acc* a) {
    return make_uint4((unsigned)__double2loint(a[0]), (unsigned)__double2hiint(a[0]),
                      (unsigned)__double2loint(a[1]), (unsigned)__double2hiint(a[1]));
  }
};
template <> struct Elem<__half> {
  static constexpr int E = 8; typedef float Acc;
  static __device__ __forceinline__ void unpack(uint4 v, Acc* a) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      a[2 * i] = f.x; a[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const Acc* a) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
      w[i] = *reinterpret_cast<const unsigned*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int E = 8; typedef float Acc;
  static __device__ __forceinline__ void unpack(uint4 v, Acc* a) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // bf16 -> fp32 is a 16-bit shift
      a[2 * i] = __uint_as_float(w[i] << 16);
      a[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const Acc* a) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
      w[i] = *reinterpret_cast<const unsigned*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <typename I> struct IntElem {
  static constexpr int E = 16 / (int)sizeof(I); typedef I Acc;
  static __device__ __forceinline__ void unpack(uint4 v, Acc* a) {
    union { uint4 v; I e[E]; } u; u.v = v;
#pragma unroll
    for (int i = 0; i < E; ++i) a[i] = u.e[i];
  }
  static __device__ __forceinline__ uint4 pack(const Acc* a) {
    union { uint4 v; I e[E]; } u;
#pragma unroll
    for (int i = 0; i < E; ++i) u.e[i] = a[i];
    return u.v;
  }
};
template <> struct Elem<uint8_t> : IntElem<uint8_t> {};
template <> struct Elem<int8_t> : IntElem<int8_t> {};
template <> struct Elem<int32_t> : IntElem<int32_t> {};
template <> struct Elem<int64_t> : IntElem<int64_t> {};

template <typename A> struct UnsignedOf { typedef A type; };
template <> struct UnsignedOf<int8_t> { typedef uint8_t type; };
template <> struct UnsignedOf<int32_t> { typedef uint32_t type; };
template <> struct UnsignedOf<int64_t> { typedef uint64_t type; };

// Integer SUM/PROD wrap modulo 2^k (computed on the unsigned twin); MIN/MAX
// use the C comparison, like MPI_MIN / MPI_MAX on the same C types.
template <int OP, typename A>
__device__ __forceinline__ A combine(A a, A b) {
  typedef typename UnsignedOf<A>::type U;
  if (OP == kProd) return (A)((U)a * (U)b);
  if (OP == kMin) return b < a ? b : a;
  if (OP == kMax) return b > a ? b : a;
  return (A)((U)a + (U)b);
}

template <typename A> __device__ __forceinline__ A apply_scale(A a, double) { return a; }
template <> __device__ __forceinline__ float apply_scale<float>(float a, double s) { return a * (float)s; }
template <> __device__ __forceinline__ double apply_scale<double>(double a, double s) { return a * s; }

// Combines x[0..n) in ascending order (x[0] first), optionally scales, packs.
template <typename T, int OP>
__device__ __forceinline__ uint4 reduce_vectors(const uint4* x, int n, bool mean, double scale) {
  typedef Elem<T> EL;
  typename EL::Acc acc[EL::E], v[EL::E];
  EL::unpack(x[0], acc);
#pragma unroll
  for (int s = 1; s < kMaxRanks; ++s) {
    if (s < n) {
      EL::unpack(x[s], v);
#pragma unroll
      for (int i = 0; i < EL::E; ++i) acc[i] = combine<OP>(acc[i], v[i]);
    }
  }
  if (mean) {
#pragma unroll
    for (int i = 0; i < EL::E; ++i) acc[i] = apply_scale(acc[i], scale);
  }
  return EL::pack(acc);
}

template <typename T>
__device__ __forceinline__ uint4 reduce_dispatch(const uint4* x, int n, int redop, double scale) {
  switch (redop) {
    case kProd: return reduce_vectors<T, kProd>(x, n, false, scale);
    case kMin: return reduce_vectors<T, kMin>(x, n, false, scale);
    case kMax: return reduce_vectors<T, kMax>(x, n, false, scale);
    case kMean: return reduce_vectors<T, kSum>(x, n, true, scale);
    default: return reduce_vectors<T, kSum>(x, n, false, scale);
  }
}

// ---------------------------------------------------------------------------
// geometry helpers

__device__ __forceinline__ char* slot_ptr(const PeerTable& pt, int owner, int parity, int b, int slot) {
  const long long idx = ((long long)parity * pt.max_blocks + b) * (pt.nranks + 1) + slot;
  return pt.stage[owner] + idx * pt.slot_bytes;
}

__device__ __forceinline__ long long clampll(long long x, long long lo, long long hi) {
  return x < lo ? lo : (x > hi ? hi : x);
}

// Start-of-launch guard and end-of-launch bookkeeping shared by all kernels.
// Epochs base+1 .. base+span belong to the launch; `done` = base + span.
struct Turn {
  u64 base;
  int parity;
};
__device__ __forceinline__ bool begin_collective(const PeerTable& pt, int b, const OpParams& P, Turn* turn) {
  const BlockState st = pt.blk[b];
  turn->base = st.epoch;
  turn->parity = (int)(st.ops & 1ull);
  return wait_peers(pt, b, st.last_done[turn->parity], P.wait_ns);
}
__device__ __forceinline__ void end_collective(const PeerTable& pt, int b, const Turn& turn, u64 done) {
  signal_peers(pt, b, done);
  if (threadIdx.x == 0) {
    BlockState* st = pt.blk + b;
    st->epoch = done;
    st->ops += 1;
    st->last_done[turn.parity] = done;
  }
}

// ---------------------------------------------------------------------------
// ALLREDUCE, one-shot: every rank stores its slice into every peer's inbox,
// one flag exchange, then every rank reduces all n copies itself (ascending
// rank order, so all ranks produce identical bits).  Epochs: +1 data, +2 done.

template <typename T, bool TABLE>
__global__ void __launch_bounds__(512, 1) ar_oneshot_kernel(const OpParams P) {
  extern __shared__ __align__(16) unsigned char smem[];
  const PeerTable& pt = P.peers[blockIdx.y];
  const RankArgs& ra = P.ra[blockIdx.y];
  const int r = pt.rank, n = pt.nranks, b = blockIdx.x;
  const Message<(int)sizeof(T), TABLE> msg = make_message<(int)sizeof(T), TABLE>(P, ra, smem);
  Turn turn;
  if (!begin_collective(pt, b, P, &turn)) return;

  const long long v0 = (long long)b * P.cv;
  const long long len = clampll(P.nvec - v0, 0, P.cv);
  char* dst[kMaxRanks];  // dst[k]: my slot in the inbox of peer (r + k) % n
#pragma unroll
  for (int k = 1; k < kMaxRanks; ++k) dst[k] = (k < n) ? slot_ptr(pt, (r + k) % n, turn.parity, b, r) : nullptr;
  for (long long v = threadIdx.x; v < len; v += blockDim.x) {
    const uint4 x = msg.load(v0 + v);
#pragma unroll
    for (int k = 1; k < kMaxRanks; ++k)
      if (k < n) stv(dst[k] + v * 16, x);
  }
  signal_peers(pt, b, turn.base + 1);
  if (!wait_peers(pt, b, turn.base + 1, P.wait_ns)) return;

  const char* const inbox0 = slot_ptr(pt, r, turn.parity, b, 0);
  for (long long v = threadIdx.x; v < len; v += blockDim.x) {
    uint4 x[kMaxRanks];
#pragma unroll
    for (int s = 0; s < kMaxRanks; ++s) {
      if (s < n) x[s] = (s == r) ? msg.load(v0 + v) : ldv(inbox0 + s * pt.slot_bytes + v * 16);
    }
    msg.store(v0 + v, reduce_dispatch<T>(x, n, P.redop, P.scale));
  }
  end_collective(pt, b, turn, turn.base + 2);
}

// ---------------------------------------------------------------------------
// ALLREDUCE two-shot / REDUCESCATTER.
// The flat message is cut into n shards of vs = ceil(nvec / n) vectors; rank r
// owns shard r.  Per round, block b works on vectors [off, off + cv) of every
// shard, off = (round * gridDim.x + b) * cv:
//   1. push   : store my copy of peer j's shard slice into j's inbox[r]
//   2. reduce : sum my shard slice over all ranks (own copy from the input,
//               the others from my inbox), scale, write to my output and to
//               my outbox
//   3. pull   : load every peer's outbox into my output
// Epochs per round i: epoch + 2i + 1 (pushed), epoch + 2i + 2 (reduced);
// done = epoch + 2 * rounds + 1.
// REDUCESCATTER (RS = true) is steps 1-2 with shard s = block s of the input
// and the result written to `out` only.

template <typename T, bool TABLE, bool RS>
__global__ void __launch_bounds__(512, 1) ar_twoshot_kernel(const OpParams P) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int ES = (int)sizeof(T);
  const PeerTable& pt = P.peers[blockIdx.y];
  const RankArgs& ra = P.ra[blockIdx.y];
  const int r = pt.rank, n = pt.nranks, b = blockIdx.x;
  const Message<ES, TABLE> msg = make_message<ES, TABLE>(P, ra, smem);
  Turn turn;
  if (!begin_collective(pt, b, P, &turn)) return;

  // Shard geometry.  AR: shards are consecutive runs of the flat message.
  // RS: shard s is the s-th block of `count` elements of the input.
  const long long vs = RS ? P.nvec : (P.nvec + n - 1) / n;
  const long long total = RS ? P.nvec * n : P.nvec;
  const char* in = static_cast<const char*>(ra.in);
  char* out = static_cast<char*>(ra.out);

  auto shard_len = [&](int s) -> long long {
    return RS ? vs : clampll(total - (long long)s * vs, 0, vs);
  };
  auto load_shard = [&](int s, long long v) -> uint4 {
    if (RS) {
      const char* base = in + (long long)s * P.count * ES;
      return load_vec<ES>(base, v, P.count, is_al16(base));
    }
    return msg.load((long long)s * vs + v);
  };

  char* const my_outbox = slot_ptr(pt, r, turn.parity, b, n);
  const char* const inbox0 = slot_ptr(pt, r, turn.parity, b, 0);
  int peer[kMaxRanks];           // peer[k] = (r + k) % n
  char* push_dst[kMaxRanks];     // my slot in peer[k]'s inbox
  const char* pull_src[kMaxRanks];  // peer[k]'s outbox
  long long plen[kMaxRanks];     // vectors in peer[k]'s shard
#pragma unroll
  for (int k = 1; k < kMaxRanks; ++k) {
    peer[k] = (k < n) ? (r + k) % n : 0;
    push_dst[k] = (k < n) ? slot_ptr(pt, peer[k], turn.parity, b, r) : nullptr;
    pull_src[k] = (k < n) ? slot_ptr(pt, peer[k], turn.parity, b, n) : nullptr;
    plen[k] = (k < n) ? shard_len(peer[k]) : 0;
  }
  for (int round = 0; round < P.rounds; ++round) {
    const long long off = ((long long)round * gridDim.x + b) * P.cv;
    const u64 e_push = turn.base + 2 * (u64)round + 1, e_red = e_push + 1;

    // 1. push
    // All loads of an iteration are issued before the first store, so a
    // thread keeps n - 1 vectors in flight.
    for (long long v = threadIdx.x; v < P.cv; v += blockDim.x) {
      uint4 x[kMaxRanks];
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k)
        if (k < n && off + v < plen[k]) x[k] = load_shard(peer[k], off + v);
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k)
        if (k < n && off + v < plen[k]) stv(push_dst[k] + v * 16, x[k]);
    }
    signal_peers(pt, b, e_push);
    if (!wait_peers(pt, b, e_push, P.wait_ns)) return;

    // 2. reduce my shard slice
    const long long mylen = clampll(shard_len(r) - off, 0, P.cv);
    for (long long v = threadIdx.x; v < mylen; v += blockDim.x) {
      uint4 x[kMaxRanks];
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < n) x[s] = (s == r) ? load_shard(r, off + v) : ldv(inbox0 + s * pt.slot_bytes + v * 16);
      }
      const uint4 y = reduce_dispatch<T>(x, n, P.redop, P.scale);
      if (RS) {
        store_vec<ES>(out, off + v, P.count, is_al16(out), y);
      } else {
        msg.store((long long)r * vs + off + v, y);
        stv(my_outbox + v * 16, y);
      }
    }
    if (RS) {
      // Peers may refill my inbox only after this read; the next round's
      // e_push wait on their side is ordered after this signal.
      signal_peers(pt, b, e_red);
      if (!wait_peers(pt, b, e_red, P.wait_ns)) return;
      continue;
    }
    signal_peers(pt, b, e_red);
    if (!wait_peers(pt, b, e_red, P.wait_ns)) return;

    // 3. pull
    for (long long v = threadIdx.x; v < P.cv; v += blockDim.x) {
      uint4 x[kMaxRanks];
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k)
        if (k < n && off + v < plen[k]) x[k] = ldv(pull_src[k] + v * 16);
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k)
        if (k < n && off + v < plen[k]) msg.store((long long)peer[k] * vs + off + v, x[k]);
    }
  }
  end_collective(pt, b, turn, turn.base + 2 * (u64)P.rounds + 1);
}

// ---------------------------------------------------------------------------
// ALLGATHER (bytes).  Per round: copy my slice to my outbox and to my own
// block of the output, signal, then pull every peer's outbox into its block
// of my output.  A second signal per round tells peers the outbox may be
// overwritten.  `count` is bytes per rank here; vectors are of bytes.

template <int kUnused>
__global__ void __launch_bounds__(512, 1) allgather_kernel(const OpParams P) {
  const PeerTable& pt = P.peers[blockIdx.y];
  const RankArgs& ra = P.ra[blockIdx.y];
  const int r = pt.rank, n = pt.nranks, b = blockIdx.x;
  Turn turn;
  if (!begin_collective(pt, b, P, &turn)) return;
  const char* in = static_cast<const char*>(ra.in);
  char* out = static_cast<char*>(ra.out);
  const bool in_al = is_al16(in);
  char* const my_outbox = slot_ptr(pt, r, turn.parity, b, n);
  int peer[kMaxRanks];
  const char* pull_src[kMaxRanks];
#pragma unroll
  for (int k = 1; k < kMaxRanks; ++k) {
    peer[k] = (k < n) ? (r + k) % n : 0;
    pull_src[k] = (k < n) ? slot_ptr(pt, peer[k], turn.parity, b, n) : nullptr;
  }

  for (int round = 0; round < P.rounds; ++round) {
    const long long off = ((long long)round * gridDim.x + b) * P.cv;
    const long long len = clampll(P.nvec - off, 0, P.cv);
    const u64 e_pub = turn.base + 2 * (u64)round + 1, e_got = e_pub + 1;
    char* mine = out + (long long)r * P.count;
    const bool mine_al = is_al16(mine);
    for (long long v = threadIdx.x; v < len; v += blockDim.x) {
      const uint4 x = load_vec<1>(in, off + v, P.count, in_al);
      stv(my_outbox + v * 16, x);
      if (mine != in) store_vec<1>(mine, off + v, P.count, mine_al, x);
    }
    signal_peers(pt, b, e_pub);
    if (!wait_peers(pt, b, e_pub, P.wait_ns)) return;
    for (long long v = threadIdx.x; v < len; v += blockDim.x) {
      uint4 x[kMaxRanks];
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k)
        if (k < n) x[k] = ldv(pull_src[k] + v * 16);
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k) {
        if (k < n) {
          char* dst = out + (long long)peer[k] * P.count;
          store_vec<1>(dst, off + v, P.count, is_al16(dst), x[k]);
        }
      }
    }
    signal_peers(pt, b, e_got);
    if (round + 1 < P.rounds && !wait_peers(pt, b, e_got, P.wait_ns)) return;
  }
  end_collective(pt, b, turn, turn.base + 2 * (u64)P.rounds + 1);
}

// ---------------------------------------------------------------------------
// BROADCAST in place (bytes).  The root publishes a slice in its outbox, the
// others pull it and acknowledge; the root refills only after all acks.

template <int kUnused>
__global__ void __launch_bounds__(512, 1) broadcast_kernel(const OpParams P) {
  const PeerTable& pt = P.peers[blockIdx.y];
  const RankArgs& ra = P.ra[blockIdx.y];
  const int r = pt.rank, n = pt.nranks, b = blockIdx.x, root = P.root;
  Turn turn;
  if (!begin_collective(pt, b, P, &turn)) return;
  char* buf = static_cast<char*>(ra.out);
  const bool al = is_al16(buf);
  char* const root_outbox = slot_ptr(pt, root, turn.parity, b, n);

  for (int round = 0; round < P.rounds; ++round) {
    const long long off = ((long long)round * gridDim.x + b) * P.cv;
    const long long len = clampll(P.nvec - off, 0, P.cv);
    const u64 e_pub = turn.base + 2 * (u64)round + 1, e_got = e_pub + 1;
    if (r == root) {
      for (long long v = threadIdx.x; v < len; v += blockDim.x)
        stv(root_outbox + v * 16, load_vec<1>(buf, off + v, P.count, al));
      signal_peers(pt, b, e_pub);
      if (round + 1 < P.rounds && !wait_peers(pt, b, e_got, P.wait_ns)) return;
    } else {
      if (!wait_peers(pt, b, e_pub, P.wait_ns, root)) return;
      for (long long v = threadIdx.x; v < len; v += blockDim.x)
        store_vec<1>(buf, off + v, P.count, al, ldv(root_outbox + v * 16));
      signal_peers(pt, b, e_got, root);
    }
  }
  end_collective(pt, b, turn, turn.base + 2 * (u64)P.rounds + 1);
}

// ---------------------------------------------------------------------------
// Single-rank path: out = in (* scale for MEAN, which is 1 at n = 1), one pass
// over HBM.  Also serves the table form (bucket -> per-tensor copies).

template <int ES, bool TABLE>
__global__ void __launch_bounds__(512, 1) local_copy_kernel(const OpParams P) {
  extern __shared__ __align__(16) unsigned char smem[];
  const Message<ES, TABLE> msg = make_message<ES, TABLE>(P, P.ra[0], smem);
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // Four independent 16-byte loads in flight per thread.
  for (; v + 3 * stride < P.nvec; v += 4 * stride) {
    const uint4 a = msg.load(v), b2 = msg.load(v + stride), c = msg.load(v + 2 * stride),
                d = msg.load(v + 3 * stride);
    msg.store(v, a); msg.store(v + stride, b2); msg.store(v + 2 * stride, c);
    msg.store(v + 3 * stride, d);
  }
  for (; v < P.nvec; v += stride) msg.store(v, msg.load(v));
}

}  // namespace dgn
