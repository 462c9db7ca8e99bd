// Device side of the sharded (ZeRO-style) AdamW step: the reduce-scatter of a
// gradient bucket, the overflow verdict, the fp32 master update on this rank's
// shard and the all-gather of the updated parameters, as two kernels.
//
// What the reference does for one bucket (dragon/operators/training/
// zero_update_op_base.cc:103-143, adam_op.cc:48-81): concat copies of all
// gradients into a flat buffer, ncclReduceScatter / MPI_Reduce_scatter,
// CheckFinite + a device-to-host read + a host all-reduce of the flag, Cast to
// fp32, Scale, Dot + Scale (clip by norm) or Clip, an optional Set per tensor
// for the learning-rate scales, the AdamW kernel, ncclAllGather /
// MPI_Allgather, split copies back into the parameters.  Here:
//
//   zero_reduce_kernel   every rank stores its copy of the other ranks' shard
//                        slices into their inboxes (remote stores); the owner
//                        sums in ascending rank order in fp32, rounds once to
//                        the element type (what the reference's receive buffer
//                        holds), widens to fp32, applies grad_scale, writes the
//                        fp32 gradient shard and leaves, per block, the sum of
//                        squares and a non-finite flag in its block state.
//   zero_update_kernel   all ranks exchange the one-bit overflow verdict
//                        through flag words (no host round trip); unless it is
//                        set, the owner clips, runs AdamW on its fp32 master
//                        shard, rounds the new values to the element type,
//                        writes them into its own parameter tensors and stores
//                        them into every peer's gather box; the peers scatter
//                        the boxes into their parameter tensors.
//
// Flat layout.  The bucket is the element-wise concatenation of its tensors
// (no padding), `total` elements; rank s owns elements [s*rc, (s+1)*rc) with
// rc = ceil(total / n), exactly the reference's partition
// (zero_update_op_base.cc:24-31).  Work is done on 16-byte vectors of the flat
// element index: vector g holds elements [g*E, g*E + E).  With tensor sizes
// that are multiples of E and 16-byte aligned tensors every access is one
// aligned vector access whatever rc is; a vector that straddles two shards is
// sent to both owners, each of which uses its own lanes only.  The fp32 state
// arrays of a rank (master, m, v, gradient shard) are indexed from the first
// vector of its shard: element e lives at index e - g_lo * E, so they stay
// vector-aligned too; the first (s*rc) % E entries are padding.
#pragma once

#include "dgn_kernels.cuh"

namespace dgn {

constexpr int kChanD = 3;

// One tensor of the bucket; `ebegin` is its first flat element.
struct ZeroEnt {
  const char* grad;
  char* param;
  long long ebegin;
  float lr_scale;
  int reserved;
};

struct ZeroRank {
  const ZeroEnt* table;  // device memory, ntensors entries
  float* master;         // fp32 copies of this rank's parameter shard
  float* m;              // first moment
  float* v;              // second moment
  float* gshard;         // reduced fp32 gradient shard (scratch between the two kernels)
  float* found_inf;      // device-visible counter, or null
};

struct ZeroParams {
  OpParams base;  // peers, wait limit, ntensors, rounds, cv
  ZeroRank zr[kMaxRanks];
  long long total;  // elements of the bucket
  long long rc;     // elements per shard, ceil(total / nranks)
  float lr, beta1, beta2, eps, wd, grad_scale, clip_norm, clip_value;
  int check_finite, use_lr_scales;
};

// Shard s in elements [e_lo, e_hi) and in vectors [g_lo, g_lo + nv).
struct ShardGeom {
  long long e_lo, e_hi, g_lo, nv;
};

__host__ __device__ inline ShardGeom shard_geom(long long total, long long rc, int s, int E) {
  ShardGeom sg;
  sg.e_lo = (long long)s * rc < total ? (long long)s * rc : total;
  sg.e_hi = sg.e_lo + rc < total ? sg.e_lo + rc : total;
  sg.g_lo = sg.e_lo / E;
  sg.nv = sg.e_hi > sg.e_lo ? (sg.e_hi + E - 1) / E - sg.g_lo : 0;
  return sg;
}

// Shared-memory footprint of the bucket table of nt tensors.
__host__ __device__ inline size_t zero_smem_bytes(int nt) {
  return (size_t)(nt + 1) * 8 + (size_t)nt * (8 + 8 + 4) + 16;
}

// The bucket table in shared memory.
template <int ES>
struct FlatBucket {
  static constexpr int E = 16 / ES;
  int nt;
  long long total;
  const long long* ebeg;     // [nt + 1], ebeg[nt] = total
  const char* const* grad;   // [nt]
  char* const* param;        // [nt]
  const float* lrs;          // [nt]

  // Tensor that holds flat element e (0 <= e < total).
  __device__ __forceinline__ int find(long long e) const {
    int lo = 0, hi = nt;  // invariant: ebeg[lo] <= e < ebeg[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (ebeg[mid] <= e) lo = mid; else hi = mid;
    }
    return lo;
  }
};

template <int ES>
__device__ __forceinline__ FlatBucket<ES> make_bucket(const ZeroParams& Z, const ZeroRank& zr, unsigned char* smem) {
  const int nt = Z.base.ntensors;
  long long* eb = reinterpret_cast<long long*>(smem);
  const char** gr = reinterpret_cast<const char**>(smem + (size_t)(nt + 1) * 8);
  char** pa = reinterpret_cast<char**>(smem + (size_t)(nt + 1) * 8 + (size_t)nt * 8);
  float* ls = reinterpret_cast<float*>(smem + (size_t)(nt + 1) * 8 + (size_t)nt * 16);
  for (int i = threadIdx.x; i < nt; i += blockDim.x) {
    const ZeroEnt e = zr.table[i];
    eb[i] = e.ebegin; gr[i] = e.grad; pa[i] = e.param; ls[i] = e.lr_scale;
  }
  if (threadIdx.x == 0) eb[nt] = Z.total;
  __syncthreads();
  FlatBucket<ES> fb;
  fb.nt = nt; fb.total = Z.total; fb.ebeg = eb; fb.grad = gr; fb.param = pa; fb.lrs = ls;
  return fb;
}

// Bytes k .. k+15 of the 32 bytes lo:hi (0 < k < 16).
__device__ __forceinline__ uint4 funnel_bytes(uint4 lo, uint4 hi, int k) {
  const unsigned w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  const int q = k >> 2;
  const unsigned sh = (unsigned)(k & 3) * 8u;
  unsigned s[5];
#pragma unroll
  for (int i = 0; i < 5; ++i) s[i] = q == 0 ? w[i] : (q == 1 ? w[i + 1] : (q == 2 ? w[i + 2] : w[i + 3]));
  return make_uint4(__funnelshift_r(s[0], s[1], sh), __funnelshift_r(s[1], s[2], sh),
                    __funnelshift_r(s[2], s[3], sh), __funnelshift_r(s[3], s[4], sh));
}

// Vector g of the flat concatenation of the tensors `ptrs` (gradients or
// parameters).  One aligned load when the vector lies inside one tensor on a
// 16-byte boundary; two aligned loads and a byte shift when it lies inside one
// tensor off the boundary; element by element across tensor borders.
// Elements at or beyond `total` read as zero.
template <int ES, typename PtrArray>
__device__ __forceinline__ uint4 flat_load(const FlatBucket<ES>& fb, PtrArray ptrs, long long g) {
  constexpr int E = 16 / ES;
  const long long e0 = g * E;
  int t = fb.find(e0);
  const long long tb = fb.ebeg[t], te = fb.ebeg[t + 1];
  const char* base = ptrs[t];
  const char* a = base + (e0 - tb) * ES;
  if (e0 + E <= te) {
    const int k = (int)(reinterpret_cast<uintptr_t>(a) & 15u);
    if (k == 0) return ldv(a);
    const char* lo = a - k;
    if (lo >= base && lo + 32 <= base + (te - tb) * ES) return funnel_bytes(ldv(lo), ldv(lo + 16), k);
  }
  typedef typename Bits<ES>::type B;
  union { uint4 v; B e[E]; } u;
  u.v = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int k = 0; k < E; ++k) {
    const long long e = e0 + k;
    if (e < fb.total) {
      while (e >= fb.ebeg[t + 1]) ++t;
      u.e[k] = __ldcg(reinterpret_cast<const B*>(ptrs[t]) + (e - fb.ebeg[t]));
    }
  }
  return u.v;
}

// Stores lanes [l0, l1) of vector g into the parameter tensors.
template <int ES>
__device__ __forceinline__ void flat_store(const FlatBucket<ES>& fb, long long g, uint4 x, int l0, int l1) {
  constexpr int E = 16 / ES;
  const long long e0 = g * E;
  int t = fb.find(e0 + l0);
  if (l0 == 0 && l1 == E && e0 + E <= fb.ebeg[t + 1]) {
    char* a = fb.param[t] + (e0 - fb.ebeg[t]) * ES;
    if (is_al16(a)) { stv(a, x); return; }
  }
  typedef typename Bits<ES>::type B;
  union { uint4 v; B e[E]; } u;
  u.v = x;
#pragma unroll
  for (int k = 0; k < E; ++k) {
    const long long e = e0 + k;
    if (k >= l0 && k < l1 && e < fb.total) {
      while (e >= fb.ebeg[t + 1]) ++t;
      __stcg(reinterpret_cast<B*>(fb.param[t]) + (e - fb.ebeg[t]), u.e[k]);
    }
  }
}

// E consecutive floats of a state array at a 16-byte aligned index.
template <int E>
__device__ __forceinline__ void load_state(const float* p, long long idx, float* out) {
#pragma unroll
  for (int q = 0; q < E / 4; ++q) {
    const float4 f = *reinterpret_cast<const float4*>(p + idx + 4 * q);
    out[4 * q] = f.x; out[4 * q + 1] = f.y; out[4 * q + 2] = f.z; out[4 * q + 3] = f.w;
  }
}
template <int E>
__device__ __forceinline__ void store_state(float* p, long long idx, const float* in, int l0, int l1) {
  if (l0 == 0 && l1 == E) {
#pragma unroll
    for (int q = 0; q < E / 4; ++q)
      *reinterpret_cast<float4*>(p + idx + 4 * q) = make_float4(in[4 * q], in[4 * q + 1], in[4 * q + 2], in[4 * q + 3]);
    return;
  }
#pragma unroll
  for (int k = 0; k < E; ++k)
    if (k >= l0 && k < l1) p[idx + k] = in[k];
}

__device__ __forceinline__ bool finite_f32(float x) { return (__float_as_uint(x) & 0x7f800000u) != 0x7f800000u; }

// ---------------------------------------------------------------------------
// Kernel 1: reduce-scatter of the gradient bucket into the fp32 gradient shard.
// Rounds, staging halves and flags are those of the lock-step two-shot kernel
// without its gather stage: pushed(i) = base+2i+1 on channel A, reduced(i) =
// base+2i+2 on channel B, done = base+2*rounds+1 on channel B.

template <typename T>
__global__ void __launch_bounds__(kMaxThreads, 1) zero_reduce_kernel(const __grid_constant__ ZeroParams Z) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float s_sq[kMaxThreads / 32];
  __shared__ int s_bad[kMaxThreads / 32];
  constexpr int ES = (int)sizeof(T);
  constexpr int E = 16 / ES;
  const OpParams& P = Z.base;
  const PeerTable& pt = P.peers[blockIdx.y];
  const ZeroRank& zr = Z.zr[blockIdx.y];
  const int r = pt.rank, n = pt.nranks, b = blockIdx.x;
  const FlatBucket<ES> fb = make_bucket<ES>(Z, zr, smem);
  Turn turn;
  if (!begin_collective(pt, b, P, &turn)) return;

  const ShardGeom mine = shard_geom(Z.total, Z.rc, r, E);
  const int rounds = P.rounds;
  const long long cv = P.cv;
  const long long stride = (long long)gridDim.x * cv;
  float sq = 0.f;
  int bad = 0;

  for (int i = 0; i <= rounds; ++i) {
    const bool do_push = i < rounds;
    const bool do_reduce = i >= 1;
    // reduced(i-2) frees the inbox half push(i) refills; pushed(i-1) publishes
    // the half reduce(i-1) reads.  Both were sent at the end of the peers'
    // previous iteration.
    if (do_push && i >= 2 && !wait_peers(pt, b, kChanB, turn.base + 2 * (u64)(i - 2) + 2, P.wait_ns)) return;
    if (do_reduce && !wait_peers(pt, b, kChanA, turn.base + 2 * (u64)(i - 1) + 1, P.wait_ns)) return;
    if (do_push) {
      const long long off = (long long)i * stride + (long long)b * cv;
      for (int k = 1; k < n; ++k) {
        const int peer = (r + 1 + (k - 1 + b) % (n - 1)) % n;  // blocks start at different peers
        const ShardGeom sg = shard_geom(Z.total, Z.rc, peer, E);
        const long long len = clampll(sg.nv - off, 0, cv);
        char* dst = slot_ptr(pt, peer, turn.parity, b, i & 1, r);
        const long long g0 = sg.g_lo + off;
        copy_vectors(len, [&](long long v) { return flat_load<ES>(fb, fb.grad, g0 + v); },
                     [&](long long v, uint4 x) { stv(dst + v * 16, x); });
      }
    }
    if (do_reduce) {
      const long long off = (long long)(i - 1) * stride + (long long)b * cv;
      const long long len = clampll(mine.nv - off, 0, cv);
      const char* inbox0 = slot_ptr(pt, r, turn.parity, b, (i - 1) & 1, 0);
      for (long long v = threadIdx.x; v < len; v += blockDim.x) {
        const long long g = mine.g_lo + off + v;
        uint4 x[kMaxRanks];
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
          if (s < n) x[s] = (s == r) ? flat_load<ES>(fb, fb.grad, g) : ldv(inbox0 + s * pt.slot_bytes + v * 16);
        }
        // Ascending rank order in fp32, one rounding to T: the value the
        // reference's receive buffer holds after its reduce-scatter.
        const uint4 y = reduce_vectors<T, kSum>(x, n, false, 1.0);
        float yf[E], d[E];
        Elem<T>::unpack(y, yf);
        const long long e0 = g * E;
        const int l0 = (int)clampll(mine.e_lo - e0, 0, E), l1 = (int)clampll(mine.e_hi - e0, 0, E);
#pragma unroll
        for (int l = 0; l < E; ++l) {
          if (l >= l0 && l < l1) {
            if (!finite_f32(yf[l])) bad = 1;
            d[l] = __fmul_rn(yf[l], Z.grad_scale);
            sq = __fmaf_rn(d[l], d[l], sq);
          } else {
            d[l] = 0.f;
          }
        }
        store_state<E>(zr.gshard, (off + v) * E, d, 0, E);
      }
    }
    if (do_push) signal_peers(pt, b, kChanA, turn.base + 2 * (u64)i + 1);
    if (do_reduce) signal_peers(pt, b, kChanB, turn.base + 2 * (u64)(i - 1) + 2);
  }

  // Per-block partials, combined in a fixed order (the same launch shape
  // always gives the same bits).
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
  }
  const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) { s_sq[warp] = sq; s_bad[warp] = bad; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float tsq = 0.f;
    int tbad = 0;
    for (int w = 0; w < nwarps; ++w) { tsq += s_sq[w]; tbad |= s_bad[w]; }
    pt.blk[b].zero_part = (u64)__float_as_uint(tsq) | ((u64)(unsigned)tbad << 32);
    if (b == 0) pt.blk[0].zero_blocks = (u64)gridDim.x;
  }
  end_collective(pt, b, turn, turn.base + 2 * (u64)rounds + 1);
}

// ---------------------------------------------------------------------------
// Kernel 2: verdict exchange, AdamW on the master shard, all-gather of the new
// parameters by remote stores.  published(i) = base+2i+1 on channel A,
// emptied(i) = base+2i+2 on channel B, done = base+2*rounds+1 on channel B.
// Channel D carries the verdict word {step count, overflow bit}: a peer cannot
// reach the next step's exchange before this rank has finished this kernel
// (the next reduce-scatter needs this rank's slices), so one word per
// (block, source) is enough.

// The reference's AdamW kernel (dragon/kernels/training/cpu/adam_kernel.cc:36-57
// and its twin with learning-rate scales in cuda/adam_kernel.cu:58-80), with
// every rounding spelled out so that no multiply-add is contracted.
__device__ __forceinline__ void adamw_lane(float g, float lr, float beta1, float beta2, float eps, float wd,
                                           float omb1, float omb2, bool scaled, float ls, float* m, float* v,
                                           float* x) {
  const float mi = __fmaf_rn(beta1, *m, __fmul_rn(omb1, g));
  const float vi = __fmaf_rn(beta2, *v, __fmul_rn(__fmul_rn(omb2, g), g));
  const float den = __fadd_rn(__fsqrt_rn(vi), eps);
  float dec;
  if (scaled) {
    const float step = __fdiv_rn(__fmul_rn(__fmul_rn(lr, ls), mi), den);
    dec = wd > 0.f ? __fmaf_rn(__fmul_rn(wd, ls), *x, step) : step;
  } else {
    const float step = __fdiv_rn(__fmul_rn(lr, mi), den);
    dec = wd > 0.f ? __fmaf_rn(wd, *x, step) : step;
  }
  *x = __fsub_rn(*x, dec);
  *m = mi;
  *v = vi;
}

template <typename T>
__global__ void __launch_bounds__(kMaxThreads, 1) zero_update_kernel(const __grid_constant__ ZeroParams Z) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float s_sumsq;
  __shared__ int s_bad;
  constexpr int ES = (int)sizeof(T);
  constexpr int E = 16 / ES;
  const OpParams& P = Z.base;
  const PeerTable& pt = P.peers[blockIdx.y];
  const ZeroRank& zr = Z.zr[blockIdx.y];
  const int r = pt.rank, n = pt.nranks, b = blockIdx.x;
  const FlatBucket<ES> fb = make_bucket<ES>(Z, zr, smem);
  Turn turn;
  if (!begin_collective(pt, b, P, &turn)) return;

  // This rank's partials of the reduce launch: warp 0 reads them strided and
  // combines them in a fixed order.
  if (threadIdx.x < 32) {
    const int nb1 = (int)pt.blk[0].zero_blocks;
    float sq = 0.f;
    int bad = 0;
    for (int j = threadIdx.x; j < nb1; j += 32) {
      const u64 w = pt.blk[j].zero_part;
      sq += __uint_as_float((unsigned)w);
      bad |= (int)(w >> 32);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      bad |= __shfl_xor_sync(0xffffffffu, bad, o);
    }
    if (threadIdx.x == 0) { s_sumsq = sq; s_bad = bad; }
  }
  const u64 tag = pt.blk[b].zero_ops + 1;
  __syncthreads();

  bool overflow = false;
  if (Z.check_finite) {
    const int t = threadIdx.x;
    const u64 word = (tag << 1) | (u64)(s_bad != 0);
    bool ok = true;
    int peer_bad = 0;
    if (t < n && t != r) {
      st_release_sys(pt.flags[t] + ((size_t)b * kChannels + kChanD) * kMaxRanks + r, word);
      const u64* f = pt.flags[r] + ((size_t)b * kChannels + kChanD) * kMaxRanks + t;
      u64 w = ld_acquire_sys(f);
      if ((w >> 1) < tag) {
        const u64 t0 = global_timer_ns();
        unsigned spins = 0;
        for (;;) {
          w = ld_acquire_sys(f);
          if ((w >> 1) >= tag) break;
          if ((++spins & 31u) == 0u && global_timer_ns() - t0 > P.wait_ns) {
            *(volatile int*)pt.status = kErrTimeout;
            ok = false;
            break;
          }
        }
      }
      peer_bad = (int)(w & 1ull);
    }
    if (!__syncthreads_and(ok)) return;
    overflow = __syncthreads_or(peer_bad | (s_bad != 0)) != 0;
    if (t == 0) {
      pt.blk[b].zero_ops = tag;
      if (b == 0 && zr.found_inf) *zr.found_inf += overflow ? 1.f : 0.f;
    }
  }

  const int rounds = P.rounds;
  if (!overflow) {
    const ShardGeom mine = shard_geom(Z.total, Z.rc, r, E);
    const long long cv = P.cv;
    const long long stride = (long long)gridDim.x * cv;
    // Clip by the L2 norm of THIS rank's shard, as the reference does
    // (zero_update_op_base.cc:90-95), else by value.
    float factor = 1.f;
    if (Z.clip_norm > 0.f) {
      const float norm = __fsqrt_rn(s_sumsq);
      if (norm > Z.clip_norm) factor = __fdiv_rn(Z.clip_norm, norm);
    }
    const bool by_value = !(Z.clip_norm > 0.f) && Z.clip_value > 0.f;
    const float omb1 = __fsub_rn(1.f, Z.beta1), omb2 = __fsub_rn(1.f, Z.beta2);
    const bool scaled = Z.use_lr_scales != 0;

    for (int i = 0; i <= rounds; ++i) {
      const bool do_update = i < rounds;
      const bool do_gather = i >= 1;
      // emptied(i-2) frees the gather-box half update(i) refills;
      // published(i-1) makes the half gather(i-1) reads complete.
      if (do_update && i >= 2 && !wait_peers(pt, b, kChanB, turn.base + 2 * (u64)(i - 2) + 2, P.wait_ns)) return;
      if (do_gather && !wait_peers(pt, b, kChanA, turn.base + 2 * (u64)(i - 1) + 1, P.wait_ns)) return;
      if (do_update) {
        const long long off = (long long)i * stride + (long long)b * cv;
        const long long len = clampll(mine.nv - off, 0, cv);
        char* gdst[kMaxRanks];  // gather box [r] of peer (r + k) % n
#pragma unroll
        for (int k = 1; k < kMaxRanks; ++k)
          gdst[k] = (k < n) ? slot_ptr(pt, (r + k) % n, turn.parity, b, i & 1, n + r) : nullptr;
        for (long long v = threadIdx.x; v < len; v += blockDim.x) {
          const long long g = mine.g_lo + off + v;
          const long long e0 = g * E, idx = (off + v) * E;
          const int l0 = (int)clampll(mine.e_lo - e0, 0, E), l1 = (int)clampll(mine.e_hi - e0, 0, E);
          float d[E], x[E], mm[E], vv[E];
          load_state<E>(zr.gshard, idx, d);
          load_state<E>(zr.master, idx, x);
          load_state<E>(zr.m, idx, mm);
          load_state<E>(zr.v, idx, vv);
          int t = scaled ? fb.find(e0 + l0) : 0;
#pragma unroll
          for (int l = 0; l < E; ++l) {
            if (l >= l0 && l < l1) {
              float gl = d[l];
              if (Z.clip_norm > 0.f) gl = __fmul_rn(gl, factor);
              else if (by_value) gl = fmaxf(-Z.clip_value, fminf(gl, Z.clip_value));
              float ls = 1.f;
              if (scaled) {
                while (e0 + l >= fb.ebeg[t + 1]) ++t;
                ls = fb.lrs[t];
              }
              adamw_lane(gl, Z.lr, Z.beta1, Z.beta2, Z.eps, Z.wd, omb1, omb2, scaled, ls, &mm[l], &vv[l], &x[l]);
            }
          }
          store_state<E>(zr.master, idx, x, l0, l1);
          store_state<E>(zr.m, idx, mm, l0, l1);
          store_state<E>(zr.v, idx, vv, l0, l1);
          const uint4 y = Elem<T>::pack(x);
          flat_store<ES>(fb, g, y, l0, l1);
#pragma unroll
          for (int k = 1; k < kMaxRanks; ++k)
            if (k < n) stv(gdst[k] + v * 16, y);
        }
      }
      if (do_gather) {
        const long long off = (long long)(i - 1) * stride + (long long)b * cv;
        for (int k = 1; k < n; ++k) {
          const int peer = (r + 1 + (k - 1 + b) % (n - 1)) % n;
          const ShardGeom sg = shard_geom(Z.total, Z.rc, peer, E);
          const long long len = clampll(sg.nv - off, 0, cv);
          const char* src = slot_ptr(pt, r, turn.parity, b, (i - 1) & 1, n + peer);
          for (long long v = threadIdx.x; v < len; v += blockDim.x) {
            const long long g = sg.g_lo + off + v;
            const long long e0 = g * E;
            const int l0 = (int)clampll(sg.e_lo - e0, 0, E), l1 = (int)clampll(sg.e_hi - e0, 0, E);
            flat_store<ES>(fb, g, ldv(src + v * 16), l0, l1);
          }
        }
      }
      if (do_update) signal_peers(pt, b, kChanA, turn.base + 2 * (u64)i + 1);
      if (do_gather) signal_peers(pt, b, kChanB, turn.base + 2 * (u64)(i - 1) + 2);
    }
  }
  end_collective(pt, b, turn, turn.base + 2 * (u64)rounds + 1);
}

// ---------------------------------------------------------------------------
// fp32 master copies of this rank's parameter shard (the reference's
// InitMaster, zero_update_op_base.cc:21-44); padding lanes become zero.
// Local work: no peer is involved.

template <typename T>
__global__ void __launch_bounds__(kMaxThreads, 1) zero_init_master_kernel(const __grid_constant__ ZeroParams Z) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int ES = (int)sizeof(T);
  constexpr int E = 16 / ES;
  const ZeroRank& zr = Z.zr[0];
  const FlatBucket<ES> fb = make_bucket<ES>(Z, zr, smem);
  const ShardGeom mine = shard_geom(Z.total, Z.rc, Z.base.peers[0].rank, E);
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < mine.nv; v += step) {
    const long long g = mine.g_lo + v;
    const long long e0 = g * E;
    const int l0 = (int)clampll(mine.e_lo - e0, 0, E), l1 = (int)clampll(mine.e_hi - e0, 0, E);
    float f[E];
    Elem<T>::unpack(flat_load<ES>(fb, fb.param, g), f);
#pragma unroll
    for (int l = 0; l < E; ++l)
      if (l < l0 || l >= l1) f[l] = 0.f;
    store_state<E>(zr.master, v * E, f, 0, E);
  }
}

}  // namespace dgn
