// solid_gpu_peer_sum_float: the sum of a pair of per-GPU partial results over the GPUs of one node, through peer
// memory.  It has no counterpart in the reference (Ocean has no collectives; its only cross-device traffic is
// cudaMemcpyPeerAsync, src/core/gpu/storage_gpu.c:140-143).  The sharded reductions end in an exchange of two floats
// per GPU; done as a library all-reduce that exchange costs 10-17 us on 2-8 GPUs, which is what bounds the scaling of
// a sub-millisecond step.  Here every GPU stores its pair straight into a slot of every peer's exchange buffer
// (plain stores over NVLink, then a release store of the step's sequence number), waits until the slots of its own
// buffer carry that number (polling its OWN memory), adds the pairs in rank order, so that every GPU computes the
// same bits, and optionally takes square roots: one block of 32 threads, one launch.
//
// The wait is bounded: a peer that does not deliver within `limit_us` makes the kernel set *status and return (the
// result is then meaningless); nothing spins without a limit.  Two sets of slots alternate with the parity of the
// sequence number, so a fast GPU's next step cannot overwrite a value a slow GPU has not read yet (it cannot be two
// steps ahead: its next exchange needs the slow GPU's contribution).
#include "solid_core_gpu.h"
#include "dtypes.cuh"
#include "layout.h"

namespace sd {

constexpr int PEER_MAX = 16;
struct PeerSumParams {
   char        *buf[PEER_MAX];
   int          world, rank, count, sqrt_mask;
   unsigned int seq;
   const float *local;
   float       *result;
   int         *status;
   unsigned long long limit_ns;
};

SD_D void st_release_sys(unsigned int *p, unsigned int v) { asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory"); }
SD_D unsigned int ld_acquire_sys(const unsigned int *p)
{  unsigned int v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
SD_D unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }

__global__ void __launch_bounds__(32) peer_sum_kernel(const PeerSumParams p)
{
   __shared__ float vals[PEER_MAX][2];
   __shared__ int failed;
   const int t = threadIdx.x;
   const size_t set = (size_t)(p.seq & 1u) * (size_t)p.world;
   if (t == 0) failed = 0;
   __syncthreads();
   if (t < p.world) {
      // my pair into slot `rank` of GPU t's buffer, then the sequence number
      char *slot = p.buf[t] + (set + (size_t)p.rank) * 16;
      const float a = p.local[0], b = p.count > 1 ? p.local[1] : 0.0f;
      asm volatile("st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" :: "l"(slot), "f"(a), "f"(b) : "memory");
      st_release_sys(reinterpret_cast<unsigned int *>(slot + 8), p.seq);
      // GPU t's pair from slot t of my own buffer
      const char *mine = p.buf[p.rank] + (set + (size_t)t) * 16;
      const unsigned long long t0 = global_ns();
      bool ok = true;
      while (ld_acquire_sys(reinterpret_cast<const unsigned int *>(mine + 8)) != p.seq) {
         if (global_ns() - t0 > p.limit_ns) { ok = false; break; }
         __nanosleep(100);
      }
      float va = 0.0f, vb = 0.0f;
      if (ok) asm volatile("ld.relaxed.sys.global.v2.f32 {%0, %1}, [%2];" : "=f"(va), "=f"(vb) : "l"(mine) : "memory");
      else failed = 1;
      vals[t][0] = va; vals[t][1] = vb;
   }
   __syncthreads();
   if (t == 0) {
      float s0 = 0.0f, s1 = 0.0f;
      for (int r = 0; r < p.world; r++) { s0 += vals[r][0]; s1 += vals[r][1]; }      // rank order on every GPU
      p.result[0] = (p.sqrt_mask & 1) ? sqrtf(s0) : s0;
      if (p.count > 1) p.result[1] = (p.sqrt_mask & 2) ? sqrtf(s1) : s1;
      if (failed && p.status != nullptr) *p.status = 1;
   }
}
} // namespace sd

extern "C" int solid_gpu_peer_sum_buffer_size(int world, size_t *size)
{
   if (size == nullptr) SD_ERROR("peer_sum_buffer_size needs a result pointer");
   if (world < 1 || world > sd::PEER_MAX) SD_ERROR("peer_sum: between 1 and %d GPUs (got %d)", sd::PEER_MAX, world);
   *size = (size_t)2 * (size_t)world * 16;                      // two sets of one 16-byte slot per GPU
   return 0;
}

extern "C" int solid_gpu_peer_sum_float(int world, int rank, void *const *buffers, unsigned int sequence, int count,
                                        const float *local, float *result, int sqrt_mask, unsigned int limit_us,
                                        int *status, cudaStream_t stream)
{
   if (world < 1 || world > sd::PEER_MAX) SD_ERROR("peer_sum: between 1 and %d GPUs (got %d)", sd::PEER_MAX, world);
   if (rank < 0 || rank >= world) SD_ERROR("peer_sum: rank %d of %d", rank, world);
   if (count < 1 || count > 2) SD_ERROR("peer_sum: one or two values per GPU (got %d)", count);
   if (sequence == 0) SD_ERROR("peer_sum: sequence numbers start at 1 (the buffers start zeroed)");
   if (buffers == nullptr || local == nullptr || result == nullptr) SD_ERROR("peer_sum: missing pointer");
   sd::PeerSumParams p;
   for (int r = 0; r < world; r++) {
      if (buffers[r] == nullptr || !sd::aligned_to(buffers[r], 16)) SD_ERROR("peer_sum: buffer %d missing or not 16-byte aligned", r);
      p.buf[r] = (char *)buffers[r];
   }
   p.world = world; p.rank = rank; p.count = count; p.sqrt_mask = sqrt_mask; p.seq = sequence;
   p.local = local; p.result = result; p.status = status;
   p.limit_ns = (unsigned long long)(limit_us ? limit_us : 2000000u) * 1000ull;      // two seconds unless told otherwise
   sd::peer_sum_kernel<<<1, 32, 0, stream>>>(p);
   SD_LAUNCH_CHECK();
   return 0;
}
