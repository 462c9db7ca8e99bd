// Gradient all-reduce fused with the optimizer update (data-parallel training
// without state sharding): every rank holds all parameters and all optimizer
// state, gradients are summed over the ranks, and every rank applies the same
// update.
//
// What the reference runs per step (torch/core/optim/optimizer.py:134-164 and
// :250-272): the `Collective` operator (ALLREDUCE, SUM) over the gradients,
// then one update operator per parameter group, whose TransformGrad
// (operators/training/update_op_base.cc:21-38) scales the summed gradient by
// grad_scale / dist_size and clips it, and whose kernel
// (kernels/training/cuda/sgd_kernel.cu:10-51, adam_kernel.cu:10-55) reads the
// gradient, the parameter and the state and writes parameter and state.  The
// summed gradient is written by the collective and read back twice.
//
// Here one kernel does all of it: the two-shot all-reduce of dgn_kernels.cuh
// (push shard slices, reduce in ascending rank order, store the reduced slice
// into the peers' gather boxes), but wherever that kernel would write a
// reduced vector into the gradient tensor, this one applies the update to the
// parameter and state vectors at the same position instead.  The summed
// gradient never goes to memory; the gradient tensors are left as they were.
// float32 gradients, parameters and state (the reference's DoRunWithTensor<float>).
//
// Every floating-point operation is spelled out with its rounding
// (__fmaf_rn / __fmul_rn / ...), in the order of the reference's kernels, so
// that parameters and state match a CPU restatement bit for bit.
#pragma once

#include "dgn_kernels.cuh"

namespace dgn {

enum : int { kUpdMomentumSGD = 0, kUpdNesterovSGD = 1, kUpdAdam = 2, kUpdAdamW = 3 };

// One tensor of the bucket: gradient, parameter, first and second state
// tensor (v is null for the SGD kinds), all of `count` floats; `vbegin` is its
// first 16-byte vector in the flat message.
struct UpdEnt {
  const char* grad;
  char* param;
  char* m;
  char* v;
  long long count;
  long long vbegin;
};

struct UpdParams {
  OpParams base;  // peers, wait limit, ntensors, nvec, rounds, cv
  const UpdEnt* table[kMaxRanks];  // device memory, ntensors entries; indexed by blockIdx.y
  int kind;
  float lr, a, b, eps, wd;  // a: momentum or beta1; b: beta2
  float grad_scale, clip_value;
};

__host__ __device__ inline size_t update_smem_bytes(int nt) {
  return (size_t)nt * (8 * 5) + (size_t)(nt + 1) * 4 + 16;
}

struct UpdBucket {
  int nt;
  const char* const* grad;
  char* const* param;
  char* const* m;
  char* const* v;
  const long long* count;
  const unsigned* vbeg;  // [nt + 1]

  __device__ __forceinline__ int find(long long vec) const {
    int lo = 0, hi = nt;  // invariant: vbeg[lo] <= vec < vbeg[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if ((long long)vbeg[mid] <= vec) lo = mid; else hi = mid;
    }
    return lo;
  }
  __device__ __forceinline__ uint4 load_grad(long long vec) const {
    const int t = find(vec);
    const char* p = grad[t];
    return load_vec<4>(p, vec - vbeg[t], count[t], is_al16(p));
  }
};

__device__ __forceinline__ UpdBucket make_update_bucket(const UpdParams& U, const UpdEnt* table, unsigned char* smem) {
  const int nt = U.base.ntensors;
  const char** g = reinterpret_cast<const char**>(smem);
  char** p = reinterpret_cast<char**>(smem + (size_t)nt * 8);
  char** m = reinterpret_cast<char**>(smem + (size_t)nt * 16);
  char** v = reinterpret_cast<char**>(smem + (size_t)nt * 24);
  long long* c = reinterpret_cast<long long*>(smem + (size_t)nt * 32);
  unsigned* vb = reinterpret_cast<unsigned*>(smem + (size_t)nt * 40);
  for (int i = threadIdx.x; i < nt; i += blockDim.x) {
    const UpdEnt e = table[i];
    g[i] = e.grad; p[i] = e.param; m[i] = e.m; v[i] = e.v; c[i] = e.count; vb[i] = (unsigned)e.vbegin;
  }
  if (threadIdx.x == 0) vb[nt] = (unsigned)U.base.nvec;
  __syncthreads();
  UpdBucket b;
  b.nt = nt; b.grad = g; b.param = p; b.m = m; b.v = v; b.count = c; b.vbeg = vb;
  return b;
}

// One element: g is the gradient summed over the ranks.
template <int KIND>
__device__ __forceinline__ void update_element(const UpdParams& U, float g, float* x, float* m, float* v) {
  if (U.grad_scale != 1.f) g = __fmul_rn(g, U.grad_scale);                    // TransformGrad: Scale
  if (U.clip_value > 0.f) g = fmaxf(-U.clip_value, fminf(g, U.clip_value));   // TransformGrad: Clip
  if (KIND == kUpdMomentumSGD || KIND == kUpdNesterovSGD) {
    const float gi = U.wd > 0.f ? __fmaf_rn(U.wd, *x, g) : g;
    const float mi = __fmaf_rn(U.a, *m, gi);
    *m = mi;
    const float step = KIND == kUpdNesterovSGD ? __fmul_rn(U.lr, __fmaf_rn(U.a, mi, gi)) : __fmul_rn(U.lr, mi);
    *x = __fsub_rn(*x, step);
  } else {
    const float gi = (KIND == kUpdAdam && U.wd > 0.f) ? __fmaf_rn(U.wd, *x, g) : g;
    const float mi = __fmaf_rn(U.a, *m, __fmul_rn(__fsub_rn(1.f, U.a), gi));
    const float vi = __fmaf_rn(U.b, *v, __fmul_rn(__fmul_rn(__fsub_rn(1.f, U.b), gi), gi));
    *m = mi;
    *v = vi;
    const float step = __fdiv_rn(__fmul_rn(U.lr, mi), __fadd_rn(__fsqrt_rn(vi), U.eps));
    const float dec = (KIND == kUpdAdamW && U.wd > 0.f) ? __fmaf_rn(U.wd, *x, step) : step;
    *x = __fsub_rn(*x, dec);
  }
}

// Applies the update to the parameter / state vectors at flat vector `vec`;
// `y` holds the four summed gradients.
template <int KIND>
__device__ __forceinline__ void update_vector(const UpdParams& U, const UpdBucket& bk, long long vec, uint4 y) {
  constexpr bool kTwo = KIND == kUpdAdam || KIND == kUpdAdamW;
  const int t = bk.find(vec);
  const long long lv = vec - bk.vbeg[t];
  const long long cnt = bk.count[t];
  char* p = bk.param[t];
  char* m = bk.m[t];
  char* v = bk.v[t];
  const bool al = is_al16(p) && is_al16(m) && (!kTwo || is_al16(v));
  const float g[4] = {__uint_as_float(y.x), __uint_as_float(y.y), __uint_as_float(y.z), __uint_as_float(y.w)};
  if (al && lv * 4 + 4 <= cnt) {
    uint4 xp = ldv(p + lv * 16), xm = ldv(m + lv * 16), xv = kTwo ? ldv(v + lv * 16) : make_uint4(0u, 0u, 0u, 0u);
    float fx[4] = {__uint_as_float(xp.x), __uint_as_float(xp.y), __uint_as_float(xp.z), __uint_as_float(xp.w)};
    float fm[4] = {__uint_as_float(xm.x), __uint_as_float(xm.y), __uint_as_float(xm.z), __uint_as_float(xm.w)};
    float fv[4] = {__uint_as_float(xv.x), __uint_as_float(xv.y), __uint_as_float(xv.z), __uint_as_float(xv.w)};
#pragma unroll
    for (int k = 0; k < 4; ++k) update_element<KIND>(U, g[k], &fx[k], &fm[k], &fv[k]);
    stv(p + lv * 16, make_uint4(__float_as_uint(fx[0]), __float_as_uint(fx[1]), __float_as_uint(fx[2]), __float_as_uint(fx[3])));
    stv(m + lv * 16, make_uint4(__float_as_uint(fm[0]), __float_as_uint(fm[1]), __float_as_uint(fm[2]), __float_as_uint(fm[3])));
    if (kTwo)
      stv(v + lv * 16, make_uint4(__float_as_uint(fv[0]), __float_as_uint(fv[1]), __float_as_uint(fv[2]), __float_as_uint(fv[3])));
    return;
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const long long e = lv * 4 + k;
    if (e < cnt) {
      float* px = reinterpret_cast<float*>(p) + e;
      float* pm = reinterpret_cast<float*>(m) + e;
      float* pv = kTwo ? reinterpret_cast<float*>(v) + e : nullptr;
      float fx = __ldcg(px), fm = __ldcg(pm), fv = kTwo ? __ldcg(pv) : 0.f;
      update_element<KIND>(U, g[k], &fx, &fm, &fv);
      __stcg(px, fx);
      __stcg(pm, fm);
      if (kTwo) __stcg(pv, fv);
    }
  }
}

// The lock-step two-shot all-reduce (ar_twoshot_kernel) with the update as its
// sink.  Iteration i runs gather(i-2), push(i) and reduce(i-1) on staging
// halves (i-2)%2, i%2, (i-1)%2; signals and waits are those of that kernel:
// pushed(i) = base+2i+1 on channel A, reduced(i) = base+2i+2 on channel B,
// done = base+2*rounds+1 on channel B.
template <int KIND>
__global__ void __launch_bounds__(kMaxThreads, 1) ar_update_kernel(const __grid_constant__ UpdParams U) {
  extern __shared__ __align__(16) unsigned char smem[];
  const OpParams& P = U.base;
  const PeerTable& pt = P.peers[blockIdx.y];
  const int r = pt.rank, n = pt.nranks, b = blockIdx.x;
  const UpdBucket bk = make_update_bucket(U, U.table[blockIdx.y], smem);
  Turn turn;
  if (!begin_collective(pt, b, P, &turn)) return;

  const long long vs = (P.nvec + n - 1) / n;
  auto shard_len = [&](int s) -> long long { return clampll(P.nvec - (long long)s * vs, 0, vs); };
  const long long mylen_total = shard_len(r);
  const int rounds = P.rounds;
  const long long cv = P.cv;
  const long long stride = (long long)gridDim.x * cv;

  for (int i = 0; i < rounds + 2; ++i) {
    const bool do_pull = i >= 2;
    const bool do_push = i < rounds;
    const bool do_reduce = i >= 1 && i <= rounds;
    if (i >= 2 && !wait_peers(pt, b, kChanB, turn.base + 2 * (u64)(i - 2) + 2, P.wait_ns)) return;
    if (do_reduce && !wait_peers(pt, b, kChanA, turn.base + 2 * (u64)(i - 1) + 1, P.wait_ns)) return;

    const long long off_push = (long long)i * stride + (long long)b * cv;
    const long long off_red = (long long)(i - 1) * stride + (long long)b * cv;
    const long long off_pull = (long long)(i - 2) * stride + (long long)b * cv;
    const long long red_len = do_reduce ? clampll(mylen_total - off_red, 0, cv) : 0;
    const char* inbox0 = slot_ptr(pt, r, turn.parity, b, (i - 1) & 1, 0);
    char* gdst[kMaxRanks];  // gather box [r] of peer (r + k) % n
#pragma unroll
    for (int k = 1; k < kMaxRanks; ++k)
      gdst[k] = (k < n) ? slot_ptr(pt, (r + k) % n, turn.parity, b, (i - 1) & 1, n + r) : nullptr;
    for (long long v0 = (long long)threadIdx.x; v0 < cv; v0 += (long long)kUnroll * blockDim.x) {
      if (do_pull) {  // gather(i-2): the peers' summed slices -> update
        for (int k = 1; k < n; ++k) {
          const int peer = (r + 1 + (k - 1 + b) % (n - 1)) % n;
          const long long len = clampll(shard_len(peer) - off_pull, 0, cv);
          const char* src = slot_ptr(pt, r, turn.parity, b, i & 1, n + peer);
          const long long obase = (long long)peer * vs + off_pull;
          uint4 x[kUnroll];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const long long v = v0 + (long long)u * blockDim.x;
            if (v < len) x[u] = ldv(src + v * 16);
          }
#pragma unroll 1
          for (int u = 0; u < kUnroll; ++u) {
            const long long v = v0 + (long long)u * blockDim.x;
            if (v < len) update_vector<KIND>(U, bk, obase + v, x[u]);
          }
        }
      }
      if (do_push) {
        for (int k = 1; k < n; ++k) {
          const int peer = (r + 1 + (k - 1 + b) % (n - 1)) % n;
          const long long len = clampll(shard_len(peer) - off_push, 0, cv);
          char* dst = slot_ptr(pt, peer, turn.parity, b, i & 1, r);
          const long long ibase = (long long)peer * vs + off_push;
          uint4 x[kUnroll];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const long long v = v0 + (long long)u * blockDim.x;
            if (v < len) x[u] = bk.load_grad(ibase + v);
          }
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const long long v = v0 + (long long)u * blockDim.x;
            if (v < len) stv(dst + v * 16, x[u]);
          }
        }
      }
      if (do_reduce) {
#pragma unroll 1
        for (int u = 0; u < kUnroll; ++u) {
          const long long v = v0 + (long long)u * blockDim.x;
          if (v < red_len) {
            uint4 x[kMaxRanks];
#pragma unroll
            for (int s = 0; s < kMaxRanks; ++s) {
              if (s < n)
                x[s] = (s == r) ? bk.load_grad((long long)r * vs + off_red + v) : ldv(inbox0 + s * pt.slot_bytes + v * 16);
            }
            const uint4 y = reduce_vectors<float, kSum>(x, n, false, 1.0);
#pragma unroll
            for (int k = 1; k < kMaxRanks; ++k)
              if (k < n) stv(gdst[k] + v * 16, y);
            update_vector<KIND>(U, bk, (long long)r * vs + off_red + v, y);
          }
        }
      }
    }
    if (do_push) signal_peers(pt, b, kChanA, turn.base + 2 * (u64)i + 1);
    if (do_reduce) signal_peers(pt, b, kChanB, turn.base + 2 * (u64)(i - 1) + 2);
  }
  end_collective(pt, b, turn, turn.base + 2 * (u64)rounds + 1);
}

}  // namespace dgn
