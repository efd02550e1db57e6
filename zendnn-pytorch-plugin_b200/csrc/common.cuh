// Shared helpers for the sm_100a kernels of libzentorch_b200: error reporting, dtype access,
// the post-op chain evaluated in the epilogue of every linear, and small PTX wrappers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/zentorch_b200.h"

namespace zt {

// ---- host-side error plumbing -----------------------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

#define ZT_REQUIRE(cond, code, ...)  \
  do {                               \
    if (!(cond)) {                   \
      ::zt::set_error(__VA_ARGS__);  \
      return (code);                 \
    }                                \
  } while (0)

#define ZT_CUDA_OK(expr)                                        \
  do {                                                          \
    cudaError_t e__ = (expr);                                   \
    if (e__ != cudaSuccess) return ::zt::cuda_fail(e__, #expr); \
  } while (0)

inline int launch_status(const char *kernel) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return cuda_fail(cudaGetLastError(), kernel);
  return ZT_SUCCESS;
}

int sm_count();

// cudaFuncSetAttribute applies to the current device only, so the "already configured" note is kept per
// device.  `done` is one flag array per kernel instantiation (a function-local static at the call site).
struct PerDeviceOnce {
  bool done[64] = {};
};
template <typename Kernel>
inline int allow_dynamic_smem(PerDeviceOnce &once, Kernel kern, int bytes) {
  int dev = 0;
  ZT_CUDA_OK(cudaGetDevice(&dev));
  ZT_REQUIRE(dev >= 0 && dev < 64, ZT_UNSUPPORTED, "device index %d out of range", dev);
  if (!once.done[dev]) {
    ZT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    once.done[dev] = true;
  }
  return ZT_SUCCESS;
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// Decode kernels are launched with programmatic stream serialisation: a kernel lets its successor start
// early (grid_launch_dependents) and itself waits for its predecessor (grid_dependency_wait) only before
// it touches what earlier work may write -- activations, scratch, output.  Weights, scales and zero points
// are read before that wait, so they must be constants of the call: a caller whose weights may have been
// written by work submitted directly before sets ZT_FLAG_WEIGHTS_VOLATILE, and the call's kernels are then
// launched with ordinary stream ordering (the wait instructions become no-ops).
// ZENTORCH_B200_PDL=0 launches everything with ordinary stream ordering.
bool overlap_launches();

// Scope of one API call: `allowed = false` (ZT_FLAG_WEIGHTS_VOLATILE) makes every launch of the call on
// this thread an ordinary stream-ordered one, so nothing is read before earlier work has completed.
class CallOverlap {
 public:
  explicit CallOverlap(bool allowed);
  ~CallOverlap();
  CallOverlap(const CallOverlap &) = delete;
  CallOverlap &operator=(const CallOverlap &) = delete;

 private:
  bool saved_;
};

#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename Kernel, typename... Args>
inline cudaError_t launch_overlapped(Kernel kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_launches() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// The same, as thread-block clusters of `cluster` CTAs (the cluster spans the grid's y dimension).
template <typename Kernel, typename... Args>
inline cudaError_t launch_overlapped_cluster(Kernel kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                             unsigned cluster_y, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = cluster_y;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_launches() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}
#endif

// ---- phase stamps for latency analysis -----------------------------------------------------------
// zt_debug_set_timeline() gives the decode kernels a device buffer; while it is set, thread 0 of every CTA
// stores %globaltimer (ns) at up to kTimelineSlots points of the kernel, one record per CTA and launch
// (records of consecutive launches follow each other; the host hands out the record offsets).  Null (the
// default) costs a uniform predicated-off branch per stamp.
constexpr int kTimelineSlots = 8;
struct TimelineSink {
  unsigned long long *base;  // null: disabled
};
TimelineSink timeline_for_launch(int ctas);   // reserves ctas * kTimelineSlots entries (or returns {nullptr})

#ifdef __CUDACC__
// by whichever single thread calls it
__device__ __forceinline__ void stamp_here(const TimelineSink &t, int cta, int slot) {
  if (t.base != nullptr) {
    unsigned long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    t.base[(size_t)cta * kTimelineSlots + slot] = ns;
  }
}
__device__ __forceinline__ void stamp(const TimelineSink &t, int cta, int slot) {
  if (threadIdx.x == 0) stamp_here(t, cta, slot);
}
#endif

// ---- post-op chain ----------------------------------------------------------------------------
struct PostOpsDev {
  int n_ops;
  int ids[ZT_MAX_POST_OPS];
  const void *bufs[ZT_MAX_POST_OPS];
};

inline PostOpsDev to_dev(const zt_post_ops_t &p) {
  PostOpsDev d{};
  d.n_ops = p.n_ops;
  for (int i = 0; i < ZT_MAX_POST_OPS; ++i) {
    d.ids[i] = p.ids[i];
    d.bufs[i] = p.buffers[i];
  }
  return d;
}

int validate_post_ops(const zt_post_ops_t &p);

__device__ __forceinline__ float bf16_bits_to_float(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }

__device__ __forceinline__ float load_as_float(const void *p, int64_t i, int dtype) {
  if (dtype == ZT_F32) return reinterpret_cast<const float *>(p)[i];
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void *p, int64_t i, int dtype, float v) {
  if (dtype == ZT_F32)
    reinterpret_cast<float *>(p)[i] = v;
  else
    reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float unary_post(float y, int id) {
  switch (id) {
    case ZT_POST_RELU: return fmaxf(y, 0.f);
    case ZT_POST_GELU_TANH: {
      const float c = 0.7978845608028654f;
      return 0.5f * y * (1.f + tanhf(c * (y + 0.044715f * y * y * y)));
    }
    case ZT_POST_GELU_ERF: return 0.5f * y * (1.f + erff(y * 0.7071067811865476f));
    case ZT_POST_SILU: return __fdividef(y, 1.f + __expf(-y));
    case ZT_POST_SIGMOID: return __fdividef(1.f, 1.f + __expf(-y));
    case ZT_POST_TANH: return tanhf(y);
    default: return y;
  }
}

// Applies the chain to one fp32 value; `idx` addresses the binary operands ([M,N] row-major, of
// dtype `buf_dtype`).
__device__ __forceinline__ float apply_post_ops(float y, const PostOpsDev &p, int64_t idx, int buf_dtype) {
  int b = 0;
#pragma unroll
  for (int i = 0; i < ZT_MAX_POST_OPS; ++i) {
    if (i < p.n_ops) {
      const int id = p.ids[i];
      if (id == ZT_POST_MUL) {
        y *= load_as_float(p.bufs[b++], idx, buf_dtype);
      } else if (id == ZT_POST_ADD) {
        y += load_as_float(p.bufs[b++], idx, buf_dtype);
      } else {
        y = unary_post(y, id);
      }
    }
  }
  return y;
}

// ---- small PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_nc_v4(const void *p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <typename T>
__host__ __device__ constexpr T ceil_div(T a, T b) {
  return (a + b - 1) / b;
}

}  // namespace zt
