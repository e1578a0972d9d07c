// Multi-GPU plumbing of the column-parallel Linear: a barrier between the ranks of one node over
// flags in each other's memory, with a BOUNDED wait, and a 2-D device-to-device copy on the copy
// engines.  The reference has no multi-device path; these have no counterpart there.
#include "common.cuh"

namespace lc {
namespace {

constexpr int kMaxRanks = 16;

struct FlagPtrs {
  uint32_t* of_rank[kMaxRanks];  // flag array (one word per rank) in rank r's memory, as mapped here
};

// Thread i tells rank i that this rank has arrived (a release store of the epoch into this rank's
// slot of rank i's array, after a system-wide fence so that everything this GPU wrote before --
// output tiles stored into peers' buffers -- is visible first), then waits until rank i's word has
// reached the epoch in this rank's own array.  The wait gives up after `budget` cycles and records
// code 4 in *status: a peer that never arrives costs a bounded delay, not a hung GPU.
__global__ void peer_barrier_kernel(FlagPtrs flags, int rank, int world, uint32_t epoch, long long budget,
                                    int32_t* status) {
  const int i = threadIdx.x;
  if (i >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.of_rank[i] + rank), "r"(epoch) : "memory");
  const uint32_t* mine = flags.of_rank[rank] + i;
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) break;  // wrap-safe "v has reached epoch"
    if (clock64() - t0 > budget) {
      if (status) atomicCAS(status, 0, 4);
      break;
    }
  }
}

}  // namespace
}  // namespace lc

using namespace lc;

extern "C" int32_t lc_peer_barrier(void* const* host_flags, int32_t rank, int32_t world, uint32_t epoch,
                                   int64_t wait_cycles, int32_t* status, void* stream) {
  if (!host_flags || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(LC_ERR_INVALID_ARG, "peer_barrier: bad rank / world (at most %d ranks)", kMaxRanks);
  if (wait_cycles <= 0) return fail(LC_ERR_INVALID_ARG, "peer_barrier: the wait must have a positive cycle budget");
  FlagPtrs f;
  for (int r = 0; r < kMaxRanks; ++r) {
    f.of_rank[r] = r < world ? static_cast<uint32_t*>(host_flags[r]) : nullptr;
    if (r < world && (!f.of_rank[r] || !aligned(f.of_rank[r], 4)))
      return fail(LC_ERR_INVALID_ARG, "peer_barrier: flag array of rank %d is null or misaligned", r);
  }
  peer_barrier_kernel<<<1, 32, 0, as_stream(stream)>>>(f, rank, world, epoch, static_cast<long long>(wait_cycles),
                                                       status);
  return check_launch("peer_barrier");
}

extern "C" int32_t lc_copy_2d_async(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch,
                                    int64_t width_bytes, int64_t rows, void* stream) {
  if (width_bytes < 0 || rows < 0 || dst_pitch < width_bytes || src_pitch < width_bytes)
    return fail(LC_ERR_INVALID_ARG, "copy_2d_async: bad shape");
  if (width_bytes == 0 || rows == 0) return LC_OK;
  if (!dst || !src) return fail(LC_ERR_INVALID_ARG, "copy_2d_async: null pointer");
  const cudaError_t err = cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch), src, static_cast<size_t>(src_pitch),
                                            static_cast<size_t>(width_bytes), static_cast<size_t>(rows),
                                            cudaMemcpyDeviceToDevice, as_stream(stream));
  if (err != cudaSuccess) return fail(LC_ERR_CUDA, "copy_2d_async: %s", cudaGetErrorString(err));
  return LC_OK;
}
