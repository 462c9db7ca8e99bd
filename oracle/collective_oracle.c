/*
 * collective_oracle.c -- CPU restatement of Dragon's `Collective` operator.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against and the CPU baseline that benchmarks time beside it.  Nothing in the
 * product (the dgn library, the Python package) may call it.
 *
 * PARITY: the 16-bit float converters and the optimizer loops below are pinned
 * to the reference's own code -- dragon/utils/conversions.h:42-149 and
 * dragon/kernels/training/cpu/{adam,sgd}_kernel.cc compile on their own behind
 * the stand-in headers of ref_stub/ (see the Makefile's `ref` target), and
 * tests/test_oracle_ref.py compares every function here with them, directly
 * and through committed vectors.  The one intended difference: a float32 above
 * the float16 range converts to infinity here (IEEE / CUDA / NCCL behaviour),
 * where conversions.h:52-54 clamps to 0x7bff.
 * The REDUCTION ORDER stays UNPINNED: the reference holds no golden vectors for
 * the collectives (test/dragon/test_distributed.py:25-52 never moves a byte
 * between ranks) and their arithmetic lives in Open MPI 4.1.2
 * (third_party/mpi/build.sh:6-12), which is absent from the reference tree and
 * from this machine.  What is restated here is therefore the operator's
 * semantics at its MPI call sites:
 *
 *   dragon/operators/distributed/collective_op.cc:37-85     operation switch,
 *       output layout of ALLGATHER ([n, *dims]) and REDUCESCATTER (dims[0]/n)
 *   dragon/operators/distributed/collective_op.cc:40-51     MEAN = SUM, then
 *       multiply by 1.f / float(comm_size)
 *   dragon/operators/distributed/collective_op.cc:89        comm_size <= 1 is a no-op
 *   dragon/operators/distributed/collective_op_impl_mpi.cc:50-85   MPI_Bcast
 *       (in place, from the group root), MPI_Allreduce, MPI_Reduce_scatter
 *       with equal counts, MPI_Allgather
 *   dragon/operators/distributed/collective_op_impl_mpi.cc:111-126 SUM/PROD/MIN/MAX
 *
 * Choices the reference leaves to the MPI library and that are fixed here:
 *   - the reduction runs over ranks in ascending order, (((x0+x1)+x2)+...);
 *     for n == 2 this is the only possible order, so fp32 SUM is bit-identical
 *     to any correct MPI_Allreduce there;
 *   - fp16 / bf16 are accumulated in fp32 and rounded once (round to nearest
 *     even, overflow to infinity, NaN -> 0x7fff).  The reference's MPI path
 *     sends them as MPI_UNSIGNED_SHORT (collective_op_impl_mpi.cc:98-99),
 *     which sums bit patterns and is numerically meaningless, so the
 *     tolerance contract for those types is against an fp64 host sum;
 *   - integer SUM wraps (two's complement), as MPI_SUM on C integers does.
 */
#define _GNU_SOURCE
#include <errno.h>
#include <math.h>
#include <sched.h>
#include <stdatomic.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <time.h>
#include <unistd.h>

enum { ORC_U8 = 0, ORC_I8, ORC_I32, ORC_I64, ORC_F16, ORC_BF16, ORC_F32, ORC_F64 };
enum { ORC_SUM = 0, ORC_MEAN, ORC_PROD, ORC_MIN, ORC_MAX };

size_t orc_dtype_size(int dtype) {
  static const size_t sz[8] = {1, 1, 4, 8, 2, 2, 4, 8};
  return (dtype >= 0 && dtype < 8) ? sz[dtype] : 0;
}

/* ---- 16-bit float conversions (IEEE-754, round to nearest even) ---------- */

float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0x1fu) {
    u = sign | 0x7f800000u | (man << 13);
  } else if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else {
    u = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t orc_f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t u = x & 0x7fffffffu;
  if (u > 0x7f800000u) return 0x7fffu;                      /* NaN */
  if (u == 0x7f800000u) return (uint16_t)(sign | 0x7c00u);  /* Inf */
  if (u >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);  /* >= 65536 */
  uint32_t result, remainder;
  if (u >= 0x38800000u) { /* normal half */
    remainder = u << 19;
    result = (u - 0x38000000u) >> 13;
  } else if (u < 0x33000000u) { /* below half of the smallest subnormal */
    return (uint16_t)sign;
  } else { /* subnormal half */
    uint32_t shift = 126u - (u >> 23); /* 14..24 */
    uint32_t man = (u & 0x7fffffu) | 0x800000u;
    remainder = man << (32u - shift);
    result = man >> shift;
  }
  if (remainder > 0x80000000u || (remainder == 0x80000000u && (result & 1u))) ++result;
  /* A carry out of the mantissa walks into the exponent, up to 0x7c00 = Inf. */
  return (uint16_t)(sign | result);
}

float orc_bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t orc_f32_to_bf16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return 0x7fffu; /* NaN */
  uint32_t remainder = x << 16;
  uint32_t result = x >> 16;
  if (remainder > 0x80000000u || (remainder == 0x80000000u && (result & 1u))) ++result;
  return (uint16_t)result;
}

/* ---- elementwise reduction over ranks ------------------------------------ */

/* One loop per reduction so that the compiler can vectorise it; the order
 * over ranks stays ascending in every loop. */
#define ORC_LOOP(T, LOAD, COMBINE, FINISH)                 \
  for (int64_t i = lo; i < hi; ++i) {                      \
    T acc = LOAD(0, i);                                    \
    for (int r = 1; r < n; ++r) {                          \
      T v = LOAD(r, i);                                    \
      COMBINE;                                             \
    }                                                      \
    FINISH;                                                \
  }
#define ORC_BY_OP(T, LOAD, SUMX, PRODX, STORE, STORE_MEAN)                \
  switch (op) {                                                           \
    case ORC_PROD: ORC_LOOP(T, LOAD, PRODX, STORE) break;                 \
    case ORC_MIN: ORC_LOOP(T, LOAD, acc = v < acc ? v : acc, STORE) break; \
    case ORC_MAX: ORC_LOOP(T, LOAD, acc = v > acc ? v : acc, STORE) break; \
    case ORC_MEAN: ORC_LOOP(T, LOAD, SUMX, STORE_MEAN) break;             \
    default: ORC_LOOP(T, LOAD, SUMX, STORE) break;                        \
  }

/* Unsigned arithmetic gives the two's-complement wraparound without UB. */
#define ORC_INT_KERNEL(NAME, T, UT)                                                            \
  static void NAME(const void* const* in, int n, int64_t lo, int64_t hi, int op, void* out) { \
    T* y = (T*)out;                                                                            \
    ORC_BY_OP(T, ORC_LOAD_##NAME, acc = (T)((UT)acc + (UT)v), acc = (T)((UT)acc * (UT)v),      \
              y[i] = acc, y[i] = acc)                                                          \
  }
#define ORC_LOAD_orc_red_u8(r, i) (((const uint8_t*)in[r])[i])
#define ORC_LOAD_orc_red_i8(r, i) (((const int8_t*)in[r])[i])
#define ORC_LOAD_orc_red_i32(r, i) (((const int32_t*)in[r])[i])
#define ORC_LOAD_orc_red_i64(r, i) (((const int64_t*)in[r])[i])

ORC_INT_KERNEL(orc_red_u8, uint8_t, uint8_t)
ORC_INT_KERNEL(orc_red_i8, int8_t, uint8_t)
ORC_INT_KERNEL(orc_red_i32, int32_t, uint32_t)
ORC_INT_KERNEL(orc_red_i64, int64_t, uint64_t)

static void orc_red_f32(const void* const* in, int n, int64_t lo, int64_t hi, int op, void* out) {
  float* y = (float*)out;
  const float scale = 1.f / (float)n;
#define ORC_LD(r, i) (((const float*)in[r])[i])
  ORC_BY_OP(float, ORC_LD, acc = acc + v, acc = acc * v, y[i] = acc, y[i] = acc * scale)
#undef ORC_LD
}

static void orc_red_f64(const void* const* in, int n, int64_t lo, int64_t hi, int op, void* out) {
  double* y = (double*)out;
  /* The reference passes the scale as a float (collective_op.cc:44-46). */
  const double scale = (double)(1.f / (float)n);
#define ORC_LD(r, i) (((const double*)in[r])[i])
  ORC_BY_OP(double, ORC_LD, acc = acc + v, acc = acc * v, y[i] = acc, y[i] = acc * scale)
#undef ORC_LD
}

static void orc_red_h(const void* const* in, int n, int64_t lo, int64_t hi, int op, void* out,
                      int bf) {
  uint16_t* y = (uint16_t*)out;
  const float scale = 1.f / (float)n;
#define ORC_LD(r, i) \
  (bf ? orc_bf16_to_f32(((const uint16_t*)in[r])[i]) : orc_f16_to_f32(((const uint16_t*)in[r])[i]))
#define ORC_ST(x) y[i] = bf ? orc_f32_to_bf16(x) : orc_f32_to_f16(x)
  ORC_BY_OP(float, ORC_LD, acc = acc + v, acc = acc * v, ORC_ST(acc), ORC_ST(acc * scale))
#undef ORC_LD
#undef ORC_ST
}

/* Reduce elements [lo, hi) of n rank buffers into out[lo, hi). */
static int orc_reduce_range(const void* const* in, int n, int64_t lo, int64_t hi, int dtype,
                            int op, void* out) {
  if (op == ORC_MEAN && dtype <= ORC_I64) return 1; /* MEAN is floating-point only */
  switch (dtype) {
    case ORC_U8: orc_red_u8(in, n, lo, hi, op, out); break;
    case ORC_I8: orc_red_i8(in, n, lo, hi, op, out); break;
    case ORC_I32: orc_red_i32(in, n, lo, hi, op, out); break;
    case ORC_I64: orc_red_i64(in, n, lo, hi, op, out); break;
    case ORC_F16: orc_red_h(in, n, lo, hi, op, out, 0); break;
    case ORC_BF16: orc_red_h(in, n, lo, hi, op, out, 1); break;
    case ORC_F32: orc_red_f32(in, n, lo, hi, op, out); break;
    case ORC_F64: orc_red_f64(in, n, lo, hi, op, out); break;
    default: return 1;
  }
  return 0;
}

/* ALLREDUCE: every rank ends with the same `count` elements (written to out). */
int orc_allreduce(const void* const* in, int n, int64_t count, int dtype, int op, void* out) {
  if (n < 1 || count < 0) return 1;
  return orc_reduce_range(in, n, 0, count, dtype, op, out);
}

/* REDUCESCATTER: each in[r] holds n*count elements; outs[r] gets block r reduced. */
int orc_reducescatter(const void* const* in, int n, int64_t count, int dtype, int op,
                      void* const* outs) {
  size_t es = orc_dtype_size(dtype);
  if (n < 1 || count < 0 || es == 0) return 1;
  for (int r = 0; r < n; ++r) {
    /* Reduce block r in place of a shifted view, then it lands at outs[r][0..count). */
    const void* shifted[64];
    for (int s = 0; s < n; ++s) shifted[s] = (const char*)in[s] + (size_t)r * count * es;
    if (orc_reduce_range(shifted, n, 0, count, dtype, op, outs[r])) return 1;
  }
  return 0;
}

/* ALLGATHER: out (identical on every rank) = concat of in[0..n) along a new dim 0. */
int orc_allgather(const void* const* in, int n, int64_t count, int dtype, void* out) {
  size_t es = orc_dtype_size(dtype);
  if (n < 1 || count < 0 || es == 0) return 1;
  for (int r = 0; r < n; ++r) memcpy((char*)out + (size_t)r * count * es, in[r], (size_t)count * es);
  return 0;
}

/* BROADCAST in place: every bufs[r] becomes a byte copy of bufs[root]. */
int orc_broadcast(void* const* bufs, int n, int64_t count, int dtype, int root) {
  size_t es = orc_dtype_size(dtype);
  if (n < 1 || root < 0 || root >= n || count < 0 || es == 0) return 1;
  for (int r = 0; r < n; ++r)
    if (r != root) memcpy(bufs[r], bufs[root], (size_t)count * es);
  return 0;
}

/* ---- MPI-shaped multi-process run (the timed CPU baseline) ----------------
 * n forked rank processes over one shared mapping, each pinned to its own
 * core when enough cores exist.  One ALLREDUCE = reduce-scatter (rank r reduces
 * shard r of all ranks' buffers in ascending rank order) + barrier + all-gather
 * (every rank copies the other shards into its own buffer), in place like
 * MPI_Allreduce(MPI_IN_PLACE, ...) at collective_op_impl_mpi.cc:62. */

typedef struct {
  atomic_int count;
  atomic_int sense;
} orc_barrier_t;

static void orc_barrier_wait(orc_barrier_t* b, int n, int* local_sense) {
  *local_sense = !*local_sense;
  if (atomic_fetch_add(&b->count, 1) == n - 1) {
    atomic_store(&b->count, 0);
    atomic_store(&b->sense, *local_sense);
  } else {
    while (atomic_load(&b->sense) != *local_sense) {
#if defined(__x86_64__)
      __builtin_ia32_pause();
#endif
    }
  }
}

static double orc_now(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

/* Runs `iters` in-place allreduces of `count` elements across n processes.
 * in[r] seeds rank r's buffer before every iteration (outside the timed
 * region).  seconds[i] receives the max-over-ranks wall time of iteration i;
 * result (may be NULL) receives rank 0's final buffer.  Returns 0 on success. */
int orc_mp_allreduce(const void* const* in, int n, int64_t count, int dtype, int op, int iters,
                     double* seconds, void* result) {
  size_t es = orc_dtype_size(dtype);
  if (n < 1 || n > 64 || count < 0 || es == 0 || iters < 1) return 1;
  size_t bytes = (size_t)count * es;
  size_t stride = (bytes + 4095) & ~(size_t)4095;
  size_t ctl = 4096 + sizeof(double) * (size_t)iters * (size_t)n;
  ctl = (ctl + 4095) & ~(size_t)4095;
  /* layout: [ctl][n work buffers][n scratch shards (one full buffer)] */
  size_t total = ctl + stride * (size_t)n + stride;
  char* shm = mmap(NULL, total, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
  if (shm == MAP_FAILED) return 2;
  orc_barrier_t* bar = (orc_barrier_t*)shm;
  atomic_init(&bar->count, 0);
  atomic_init(&bar->sense, 0);
  double* times = (double*)(shm + 4096);
  char* work = shm + ctl;
  char* scratch = work + stride * (size_t)n;
  long ncores = sysconf(_SC_NPROCESSORS_ONLN);

  pid_t pids[64];
  for (int r = 0; r < n; ++r) {
    pid_t pid = fork();
    if (pid < 0) return 3;
    if (pid == 0) {
      if (ncores >= n) {
        cpu_set_t set;
        CPU_ZERO(&set);
        CPU_SET(r % ncores, &set);
        sched_setaffinity(0, sizeof(set), &set);
      }
      int sense = 0;
      int64_t per = (count + n - 1) / n;
      int64_t lo = per * r < count ? per * r : count;
      int64_t hi = lo + per < count ? lo + per : count;
      const void* bufs[64];
      for (int s = 0; s < n; ++s) bufs[s] = work + stride * (size_t)s;
      for (int it = 0; it < iters; ++it) {
        memcpy(work + stride * (size_t)r, in[r], bytes);
        orc_barrier_wait(bar, n, &sense);
        double t0 = orc_now();
        /* reduce-scatter: shard r of every rank, ascending rank order */
        orc_reduce_range(bufs, n, lo, hi, dtype, op, scratch);
        orc_barrier_wait(bar, n, &sense);
        /* all-gather: pull every reduced shard into this rank's buffer */
        memcpy(work + stride * (size_t)r, scratch, bytes);
        orc_barrier_wait(bar, n, &sense);
        times[(size_t)it * n + r] = orc_now() - t0;
      }
      _exit(0);
    }
    pids[r] = pid;
  }
  int bad = 0;
  for (int r = 0; r < n; ++r) {
    int st = 0;
    if (waitpid(pids[r], &st, 0) < 0 || !WIFEXITED(st) || WEXITSTATUS(st) != 0) bad = 1;
  }
  if (!bad) {
    for (int it = 0; it < iters; ++it) {
      double m = 0;
      for (int r = 0; r < n; ++r)
        if (times[(size_t)it * n + r] > m) m = times[(size_t)it * n + r];
      seconds[it] = m;
    }
    if (result) memcpy(result, work, bytes);
  }
  munmap(shm, total);
  return bad ? 4 : 0;
}

/* ---- AdamW on an fp32 shard (the update of the sharded optimizer step) -------
 * Restates the reference's CPU kernel _AdamW
 * (dragon/kernels/training/cpu/adam_kernel.cc:36-57) and, when `lrs` is given,
 * its variant with per-element learning-rate scales
 * (dragon/kernels/training/cuda/adam_kernel.cu:58-80; that variant has no CPU
 * twin in the reference).  x and y are the same array there (the fp32 master
 * copy, zero_update_op_base.cc:139 with adam_op.cc:58-62), so one pointer is
 * taken here.  `lr` and `wd` are what the operator passes: lr * correction and
 * lr * weight_decay (adam_op.cc:52,56).  Built with -ffp-contract=off: every
 * operation below rounds exactly once, fmaf is the only fused one. */
void orc_adamw(int64_t n, float lr, float beta1, float beta2, float eps, float wd, const float* lrs,
               const float* g, float* m, float* v, float* y) {
  for (int64_t i = 0; i < n; ++i) {
    const float gi = g[i];
    const float mi = m[i] = fmaf(beta1, m[i], (1.f - beta1) * gi);
    const float vi = v[i] = fmaf(beta2, v[i], (1.f - beta2) * gi * gi);
    if (lrs) {
      y[i] -= wd > 0.f ? fmaf(wd * lrs[i], y[i], lr * lrs[i] * mi / (sqrtf(vi) + eps))
                       : lr * lrs[i] * mi / (sqrtf(vi) + eps);
    } else {
      y[i] -= wd > 0.f ? fmaf(wd, y[i], lr * mi / (sqrtf(vi) + eps)) : lr * mi / (sqrtf(vi) + eps);
    }
  }
}

/* Adam with coupled weight decay (dragon/kernels/training/cuda/adam_kernel.cu:10-31,
 * CPU twin cpu/adam_kernel.cc:11-32): x is the parameter before the step; the
 * callers here pass x == y, as the update operators do. */
void orc_adam(int64_t n, float lr, float beta1, float beta2, float eps, float wd, const float* g, float* m,
              float* v, float* y) {
  for (int64_t i = 0; i < n; ++i) {
    const float gi = wd > 0.f ? fmaf(wd, y[i], g[i]) : g[i];
    const float mi = m[i] = fmaf(beta1, m[i], (1.f - beta1) * gi);
    const float vi = v[i] = fmaf(beta2, v[i], (1.f - beta2) * gi * gi);
    y[i] -= lr * mi / (sqrtf(vi) + eps);
  }
}

/* SGD with momentum, plain or Nesterov (dragon/kernels/training/cuda/sgd_kernel.cu:10-51,
 * CPU twin cpu/sgd_kernel.cc:10-45). */
void orc_momentum_sgd(int64_t n, float lr, float momentum, float wd, int nesterov, const float* g, float* m,
                      float* y) {
  for (int64_t i = 0; i < n; ++i) {
    const float gi = wd > 0.f ? fmaf(wd, y[i], g[i]) : g[i];
    const float mi = m[i] = fmaf(momentum, m[i], gi);
    y[i] -= nesterov ? lr * fmaf(momentum, mi, gi) : lr * mi;
  }
}
