// One-shot all-reduce of a small bf16 tensor over peer memory: the collective after a row-parallel decode
// linear.
//
// At decode sizes (16 KB to 1 MB) an all-reduce is pure latency: a library call costs 10 to 15 microseconds
// per collective, several times the linear it follows.  Here every GPU owns a symmetric buffer that its peers
// can address (the caller allocates it and passes everybody's base pointers), with one slot per source rank.
// The kernel pushes its partial sums into its slot of every peer's buffer over NVLink as 8-byte words, each
// holding 4 bytes of data and the number of the call: an aligned 8-byte store arrives whole, so the receiver
// needs no separate flag and the sender no fence -- it polls the words of its own buffer (local reads that do
// not use L1) until each carries this call's number, and adds the data in rank order in fp32.  Every rank
// computes the same sum in the same order, so the results are identical on all ranks.  One NVLink crossing
// lies on the critical path.  No multimem, no TMA to or from peer memory, nothing but ld / st.
//
// Words travel two at a time (st.v2.u64: two 8-byte elements, each whole) and a slot is laid out in two planes,
// plane j holding words 2j and 2j + 1 of every 16-byte input vector, so that the lanes of a warp write
// consecutive 16-byte pieces: 512 contiguous bytes per store instruction instead of 32 scattered 8-byte ones.
//
// Work is cut into independent slices, one per CTA, so there is no grid-wide step.  Calls are numbered by an
// epoch kept in this GPU's memory and advanced by the kernel itself (by the last CTA to finish, so that every
// CTA of a launch reads the same number), which makes a captured launch replayable.  A word's number is that
// of its last writer, which is older than the current call by a multiple of two: stale words never look
// current.  Two buffers alternate with the epoch, which is enough: a peer pushes the data of call e + 2
// (same buffer as call e) only after it has seen this rank's words of call e + 1, which this rank sends after
// it has finished reading call e.
#include "tc05.cuh"

namespace zt {

namespace {

constexpr int kArThreads = 256;
constexpr int kStatusPeerTimeout = 105;   // a peer's words did not arrive within the poll limit

struct ArParams {
  const uint4 *in;
  uint4 *out;
  long long vecs;          // 16-byte vectors in the tensor
  long long slice_vecs;    // per CTA
  unsigned char *base[ZT_AR_MAX_RANKS];
  int rank, world;
  size_t slot_bytes, buf_bytes;   // a buffer is one slot per source rank; a slot holds twice the tensor's bytes
  uint32_t *epochs;
  int *status;
};

// two {data, call number} words as one 16-byte access of two 8-byte elements
__device__ __forceinline__ void st_pair(void *p, uint32_t d0, uint32_t d1, uint32_t epoch) {
  const unsigned long long w0 = (unsigned long long)d0 | ((unsigned long long)epoch << 32);
  const unsigned long long w1 = (unsigned long long)d1 | ((unsigned long long)epoch << 32);
  asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(w0), "l"(w1) : "memory");
}
__device__ __forceinline__ void ld_pair(const void *p, unsigned long long &w0, unsigned long long &w1) {
  asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(p) : "memory");
}

__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const ArParams p) {
  __shared__ int s_ok;
  const int cta = blockIdx.x, tid = threadIdx.x;
  grid_launch_dependents();
  if (tid == 0) s_ok = 1;
  const long long v0 = (long long)cta * p.slice_vecs;
  const long long v1 = min(p.vecs, v0 + p.slice_vecs);
  // The partial sums come from the preceding kernel, and the epoch word from the previous call of this kernel,
  // which has certainly completed only once the kernels between it and this one have.
  grid_dependency_wait();
  const uint32_t epoch = p.epochs[0] + 1;                   // this call's number (own memory)
  const size_t buf_off = (size_t)(epoch & 1) * p.buf_bytes;
  const size_t my_slot = buf_off + (size_t)p.rank * p.slot_bytes;
  const size_t plane = p.slot_bytes / 2;                    // bytes of one plane of a slot
  __syncthreads();
  bool ok = true;
  for (long long i = v0 + tid; i < v1; i += kArThreads) {
    const uint4 mine = p.in[i];
    // 1. push: two 16-byte pieces per 16 bytes of data into my slot of every peer's buffer
#pragma unroll
    for (int r = 0; r < ZT_AR_MAX_RANKS; ++r)
      if (r < p.world && r != p.rank) {
        unsigned char *dst = p.base[r] + my_slot + (size_t)i * 16;
        st_pair(dst, mine.x, mine.y, epoch);
        st_pair(dst + plane, mine.z, mine.w, epoch);
      }
    // 2. collect: the same pieces of every peer's slot in my buffer, once they carry this call's number
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < ZT_AR_MAX_RANKS; ++r)
      if (r < p.world) {
        uint32_t d[4] = {mine.x, mine.y, mine.z, mine.w};
        if (r != p.rank) {
          const unsigned char *src = p.base[p.rank] + buf_off + (size_t)r * p.slot_bytes + (size_t)i * 16;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            unsigned long long w0, w1;
            ld_pair(src + j * plane, w0, w1);
            for (uint32_t spin = 0; ((uint32_t)(w0 >> 32) != epoch || (uint32_t)(w1 >> 32) != epoch) && ok; ++spin) {
              if (spin >= tc::kSpinLimit) {
                ok = false;
                break;
              }
              if (spin > 64) __nanosleep(50);
              ld_pair(src + j * plane, w0, w1);
            }
            d[2 * j] = (uint32_t)w0;
            d[2 * j + 1] = (uint32_t)w1;
          }
        }
        // 3. the sum, in rank order on every rank
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += __uint_as_float(d[j] << 16);
          acc[2 * j + 1] += __uint_as_float(d[j] & 0xffff0000u);
        }
      }
    if (ok) {
      uint4 o;
      __nv_bfloat162 t0 = __floats2bfloat162_rn(acc[0], acc[1]), t1 = __floats2bfloat162_rn(acc[2], acc[3]);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[4], acc[5]), t3 = __floats2bfloat162_rn(acc[6], acc[7]);
      o.x = *reinterpret_cast<uint32_t *>(&t0);
      o.y = *reinterpret_cast<uint32_t *>(&t1);
      o.z = *reinterpret_cast<uint32_t *>(&t2);
      o.w = *reinterpret_cast<uint32_t *>(&t3);
      p.out[i] = o;
    }
  }
  if (!ok) {
    tc::report_timeout(p.status, kStatusPeerTimeout);
    s_ok = 0;
  }
  __syncthreads();
  // the last CTA to finish advances the call number: by then every CTA of this launch has read it
  if (tid == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(&p.epochs[1], 1u);
    if (done == gridDim.x - 1) {
      p.epochs[1] = 0;
      __threadfence();
      p.epochs[0] = epoch;
    }
  }
}


}  // namespace
}  // namespace zt

using namespace zt;

extern "C" size_t zt_allreduce_symmetric_bytes(size_t max_bytes) {
  const size_t slot = 2 * ((max_bytes + 255) / 256 * 256);   // every 4 bytes of data travel with the call number
  return 2 * ZT_AR_MAX_RANKS * slot;                         // two buffers of one slot per source rank
}

extern "C" int zt_allreduce_bf16(const zt_allreduce_args_t *a, void *stream) {
  ZT_REQUIRE(a != nullptr, ZT_INVALID_ARGUMENT, "zt_allreduce_bf16: null argument block");
  ZT_REQUIRE(a->world >= 1 && a->world <= ZT_AR_MAX_RANKS && a->rank >= 0 && a->rank < a->world, ZT_INVALID_ARGUMENT,
             "zt_allreduce_bf16: rank %d of %d (at most %d ranks)", a->rank, a->world, ZT_AR_MAX_RANKS);
  ZT_REQUIRE(a->numel >= 0, ZT_INVALID_ARGUMENT, "zt_allreduce_bf16: negative size");
  if (a->numel == 0) return ZT_SUCCESS;
  ZT_REQUIRE(a->in && a->out && a->epochs, ZT_INVALID_ARGUMENT, "zt_allreduce_bf16: null pointer");
  ZT_REQUIRE(a->numel % 8 == 0 && ((reinterpret_cast<uintptr_t>(a->in) | reinterpret_cast<uintptr_t>(a->out)) & 15) == 0,
             ZT_UNSUPPORTED, "zt_allreduce_bf16: the tensor must be a multiple of 8 elements and 16-byte aligned");
  const size_t bytes = (size_t)a->numel * 2;
  ZT_REQUIRE(bytes <= a->max_bytes, ZT_UNSUPPORTED,
             "zt_allreduce_bf16: %zu bytes exceed the symmetric buffer's %zu; use the library collective", bytes,
             a->max_bytes);
  ArParams p{};
  for (int r = 0; r < a->world; ++r) {
    ZT_REQUIRE(a->peer_base[r] != nullptr && (reinterpret_cast<uintptr_t>(a->peer_base[r]) & 255) == 0, ZT_INVALID_ARGUMENT,
               "zt_allreduce_bf16: peer base %d must be a 256-byte aligned pointer", r);
    p.base[r] = reinterpret_cast<unsigned char *>(a->peer_base[r]);
  }
  p.in = reinterpret_cast<const uint4 *>(a->in);
  p.out = reinterpret_cast<uint4 *>(a->out);
  p.vecs = a->numel / 8;
  p.rank = a->rank;
  p.world = a->world;
  p.slot_bytes = 2 * ((a->max_bytes + 255) / 256 * 256);
  p.buf_bytes = ZT_AR_MAX_RANKS * p.slot_bytes;
  p.epochs = a->epochs;
  p.status = device_status_ptr();
  // slices of at least 4 KB (256 vectors), at most ZT_AR_MAX_SLICES of them; the count must depend on the size
  // only, so that every rank cuts the tensor the same way
  long long slices = (p.vecs + 255) / 256;
  if (slices > ZT_AR_MAX_SLICES) slices = ZT_AR_MAX_SLICES;
  p.slice_vecs = (p.vecs + slices - 1) / slices;
  slices = (p.vecs + p.slice_vecs - 1) / p.slice_vecs;
  ZT_CUDA_OK(launch_overlapped(allreduce_oneshot_kernel, dim3((unsigned)slices), dim3(kArThreads), (size_t)0,
                               (cudaStream_t)stream, p));
  return launch_status("allreduce_oneshot_kernel");
}
