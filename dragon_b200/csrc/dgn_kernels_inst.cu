// One translation unit per element type (DGN_INST selects it) so the
// template instantiations compile in parallel.  Each unit exports the host
// stubs of its kernels as plain function pointers.
#include "dgn_kernels.cuh"

#ifndef DGN_INST
#error "compile with -DDGN_INST=<dtype index 0..7, or 8 for the byte kernels>"
#endif

namespace dgn {

#if DGN_INST == 0
typedef uint8_t InstT;
#elif DGN_INST == 1
typedef int8_t InstT;
#elif DGN_INST == 2
typedef int32_t InstT;
#elif DGN_INST == 3
typedef int64_t InstT;
#elif DGN_INST == 4
typedef __half InstT;
#elif DGN_INST == 5
typedef __nv_bfloat16 InstT;
#elif DGN_INST == 6
typedef float InstT;
#elif DGN_INST == 7
typedef double InstT;
#endif

#define DGN_CAT2(a, b) a##b
#define DGN_CAT(a, b) DGN_CAT2(a, b)

#if DGN_INST < 8
// kind: 0 one-shot, 1 two-shot (lock-step), 2 reduce-scatter, 3 low-latency one-shot,
//       4 two-shot (warp-specialised), 5 low-latency two-shot,
//       6 staged ring through NVSwitch multicast (float, half and bfloat16 only),
//       7 NVSwitch multicast in place on symmetric memory (the same types),
//       8 staged ring with peer loads and stores (every type)
const void* DGN_CAT(reduce_kernel_fn_, DGN_INST)(int kind, bool table) {
  switch (kind) {
    case 0:
      return table ? (const void*)ar_oneshot_kernel<InstT, true>
                   : (const void*)ar_oneshot_kernel<InstT, false>;
    case 1:
      return table ? (const void*)ar_twoshot_kernel<InstT, true, false>
                   : (const void*)ar_twoshot_kernel<InstT, false, false>;
    case 2:
      return (const void*)ar_twoshot_kernel<InstT, false, true>;
    case 4:
      return table ? (const void*)ar_twoshot_ws_kernel<InstT, true>
                   : (const void*)ar_twoshot_ws_kernel<InstT, false>;
#if DGN_INST >= 4 && DGN_INST <= 6
    case 6:
      return table ? (const void*)ar_flow_kernel<InstT, true, true>
                   : (const void*)ar_flow_kernel<InstT, false, true>;
    case 7:
      return table ? nullptr : (const void*)ar_nvls_inplace_kernel<InstT>;
#endif
    case 8:
      return table ? (const void*)ar_flow_kernel<InstT, true, false>
                   : (const void*)ar_flow_kernel<InstT, false, false>;
    case 5:
      return table ? (const void*)ar_twoshot_ll_kernel<InstT, true>
                   : (const void*)ar_twoshot_ll_kernel<InstT, false>;
    case 3:
      return table ? (const void*)ar_oneshot_ll_kernel<InstT, true>
                   : (const void*)ar_oneshot_ll_kernel<InstT, false>;
    default:
      return nullptr;
  }
}
#else
const void* allgather_kernel_fn() { return (const void*)allgather_kernel<0>; }
const void* allgather_pull_kernel_fn() { return (const void*)allgather_pull_kernel<0>; }
const void* allgather_ll_kernel_fn() { return (const void*)allgather_ll_kernel<0>; }
const void* broadcast_kernel_fn() { return (const void*)broadcast_kernel<0>; }
const void* broadcast_scatter_kernel_fn() { return (const void*)broadcast_scatter_kernel<0>; }
const void* gather_flow_kernel_fn(bool through_switch) {
  return through_switch ? (const void*)gather_flow_kernel<true> : (const void*)gather_flow_kernel<false>;
}
const void* local_copy_kernel_fn(int es, bool table) {
  switch (es) {
    case 1: return table ? (const void*)local_copy_kernel<1, true> : (const void*)local_copy_kernel<1, false>;
    case 2: return table ? (const void*)local_copy_kernel<2, true> : (const void*)local_copy_kernel<2, false>;
    case 4: return table ? (const void*)local_copy_kernel<4, true> : (const void*)local_copy_kernel<4, false>;
    case 8: return table ? (const void*)local_copy_kernel<8, true> : (const void*)local_copy_kernel<8, false>;
    default: return nullptr;
  }
}
#endif

}  // namespace dgn
