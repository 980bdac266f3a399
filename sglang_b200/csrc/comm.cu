// Peer-memory plumbing and the second half of the fused row-parallel all-reduce, for sm_100a over NVLink.
//
// A row-parallel layer ends in a sum over the tensor-parallel ranks.  Here that sum is a two-shot all-reduce
// whose first shot is folded into the GEMM: the GEMM's epilogue stores every output tile straight into the
// staging buffer of the rank that owns those rows (sglb200_fp8_blockwise_scaled_mm_push), so the
// reduce-scatter traffic crosses NVLink while later tiles are still being computed.  The kernel in this file
// is the rest: wait until every rank's GEMM has finished, add the `world` partial blocks of the rows this
// rank owns in rank order (float32, one rounding: every rank ends up with bit-identical rows), then fetch the
// other ranks' reduced rows with plain peer loads.
//
// Buffers that peers touch are ordinary cudaMalloc memory exported with CUDA IPC handles (the scheme of the
// reference's custom all-reduce, sgl-kernel/csrc/allreduce/custom_all_reduce.cuh).  Ranks synchronise inside
// the kernel through flag words in each other's memory; every wait is bounded and ends in a status word.
// One process drives one GPU, so the waiting kernels of different ranks never share a GPU.
#include <cstring>

#include "common.cuh"

namespace sglb200 {

constexpr int kCommThreads = 512;
constexpr int kCommMaxBlocks = 148;
constexpr int kCommMaxWorld = 8;
constexpr unsigned kCommSpinLimit = 1u << 22;  // default probes of about 0.25 us each: around a second

__device__ int g_comm_status = 0;  // 0 ok, 1 = a wait for a peer's flag expired

struct CommPeers {
  const uint16_t* stage;               // this rank's staging buffer [world][rows_own][N]
  uint16_t* reduced[kCommMaxWorld];    // every rank's buffer of reduced rows [rows_own][N]
  uint32_t* flags[kCommMaxWorld];      // every rank's flag words [2][kCommMaxBlocks][kCommMaxWorld], then this
                                       // rank's own call counters [kCommMaxBlocks]
  unsigned spin_limit;                 // probes after which a wait for a peer gives up
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The epoch of a call lives on the device: block b of a rank counts its own calls in a word of the rank's flag
// buffer that only it touches.  Every rank launches the same sequence of calls with the same grid, so block b
// of every rank reads the same number, and a CUDA graph that replays a call gets a fresh epoch on every replay
// (a host-side counter would be frozen into the graph).  0 is the cleared state of the flags and is skipped.
__device__ __forceinline__ uint32_t next_epoch(const CommPeers& c, int rank, uint32_t* s_epoch) {
  if (threadIdx.x == 0) {
    uint32_t* counter = c.flags[rank] + (size_t)2 * kCommMaxBlocks * kCommMaxWorld + blockIdx.x;
    uint32_t e = *counter + 1u;
    if (e == 0u) e = 1u;
    *counter = e;
    *s_epoch = e;
  }
  __syncthreads();
  return *s_epoch;
}

// Block-level barrier across the ranks: block b of every rank tells block b of every other rank that it has
// arrived (flag = epoch) and waits for theirs.  `phase` selects the flag set.  Returns false if a peer never
// showed up; the caller then leaves without touching peer data.
__device__ __forceinline__ bool cross_rank_barrier(const CommPeers& c, int world, int rank, int phase, uint32_t epoch,
                                                   int* s_ok) {
  __syncthreads();  // this block's earlier writes are done ...
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    const size_t slot = ((size_t)phase * kCommMaxBlocks + blockIdx.x) * kCommMaxWorld;
    __threadfence_system();  // ... and ordered before the flag for whoever acquires it
    st_release_sys(c.flags[peer] + slot + rank, epoch);
    const uint32_t* mine = c.flags[rank] + slot + peer;
    unsigned n = 0;
    while (ld_acquire_sys(mine) != epoch) {
      if (++n > c.spin_limit) {
        *s_ok = 0;
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  return *s_ok != 0;
}

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

template <bool kFp16>
__device__ __forceinline__ void add_packed(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (kFp16) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      acc[2 * i] += f.x, acc[2 * i + 1] += f.y;
    } else {
      acc[2 * i] += bf16lo(w[i]), acc[2 * i + 1] += bf16hi(w[i]);
    }
  }
}

// out [M][N]: this rank's private result.  chunks = rows_per_owner * N / 8 (16-byte pieces per owner's block of rows),
// total_chunks = M * N / 8: owner d holds the pieces [d * chunks, min((d + 1) * chunks, total_chunks)).
template <bool kFp16>
__global__ void __launch_bounds__(kCommThreads)
    reduce_gather_kernel(CommPeers c, uint16_t* __restrict__ out, int64_t chunks, int64_t total_chunks, int world,
                         int rank) {
  __shared__ int s_ok;
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) s_ok = 1;
  const uint32_t epoch = next_epoch(c, rank, &s_epoch);
  if (!cross_rank_barrier(c, world, rank, 0, epoch, &s_ok)) {
    if (threadIdx.x == 0) atomicExch(&g_comm_status, 1);
    return;
  }
  // every rank's GEMM has finished: the `world` partial blocks of my rows are complete in my staging buffer
  const uint4* stage = reinterpret_cast<const uint4*>(c.stage);
  uint4* mine = reinterpret_cast<uint4*>(c.reduced[rank]);
  uint4* out4 = reinterpret_cast<uint4*>(out);
  const int64_t stride = (int64_t)gridDim.x * kCommThreads;
  auto owned = [&](int d) {  // pieces of owner d's block that lie inside the output
    const int64_t left = total_chunks - (int64_t)d * chunks;
    return left < 0 ? (int64_t)0 : (left < chunks ? left : chunks);
  };
  const int64_t my_chunks = owned(rank);
  for (int64_t i = (int64_t)blockIdx.x * kCommThreads + threadIdx.x; i < my_chunks; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 v[kCommMaxWorld];
#pragma unroll
    for (int s = 0; s < kCommMaxWorld; ++s)
      if (s < world) v[s] = stage[(int64_t)s * chunks + i];
#pragma unroll
    for (int s = 0; s < kCommMaxWorld; ++s)
      if (s < world) add_packed<kFp16>(acc, v[s]);  // rank order: the same sum on every run
    uint4 r;
    uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (kFp16) {
        const __half2 h = __floats2half2_rn(acc[2 * k], acc[2 * k + 1]);
        rw[k] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
        rw[k] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    mine[i] = r;
    out4[(int64_t)rank * chunks + i] = r;
  }
  if (!cross_rank_barrier(c, world, rank, 1, epoch, &s_ok)) {
    if (threadIdx.x == 0) atomicExch(&g_comm_status, 1);
    return;
  }
  // every rank's reduced rows are complete: fetch the others', starting with the next rank so that the ranks
  // do not all read from the same peer at once
  for (int d = 1; d < world; ++d) {
    const int peer = (rank + d) % world;
    const uint4* src = reinterpret_cast<const uint4*>(c.reduced[peer]);
    uint4* dst = out4 + (int64_t)peer * chunks;
    const int64_t peer_chunks = owned(peer);
    int64_t i = (int64_t)blockIdx.x * kCommThreads + threadIdx.x;
    constexpr int kFlight = 8;  // peer loads in flight per thread: a small grid must still cover the NVLink latency
    for (; i + (kFlight - 1) * stride < peer_chunks; i += kFlight * stride) {
      uint4 v[kFlight];
#pragma unroll
      for (int k = 0; k < kFlight; ++k) v[k] = src[i + k * stride];
#pragma unroll
      for (int k = 0; k < kFlight; ++k) dst[i + k * stride] = v[k];
    }
    for (; i < peer_chunks; i += stride) dst[i] = src[i];
  }
}

}  // namespace sglb200

using namespace sglb200;

extern "C" int sglb200_comm_alloc(int64_t bytes, void** out) {
  SGLB_REQUIRE(bytes > 0 && out != nullptr, "comm_alloc: bad arguments");
  void* p = nullptr;
  SGLB_CUDA(cudaMalloc(&p, (size_t)bytes));
  SGLB_CUDA(cudaMemset(p, 0, (size_t)bytes));
  SGLB_CUDA(cudaDeviceSynchronize());
  *out = p;
  return SGLB200_OK;
}

extern "C" int sglb200_comm_free(void* p) {
  if (p != nullptr) SGLB_CUDA(cudaFree(p));
  return SGLB200_OK;
}

extern "C" int sglb200_comm_ipc_export(void* p, void* handle64) {
  SGLB_REQUIRE(p != nullptr && handle64 != nullptr, "comm_ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  SGLB_CUDA(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p));
  return SGLB200_OK;
}

extern "C" int sglb200_comm_ipc_open(const void* handle64, void** out) {
  SGLB_REQUIRE(handle64 != nullptr && out != nullptr, "comm_ipc_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  SGLB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return SGLB200_OK;
}

extern "C" int sglb200_comm_ipc_close(void* p) {
  if (p != nullptr) SGLB_CUDA(cudaIpcCloseMemHandle(p));
  return SGLB200_OK;
}

extern "C" int64_t sglb200_comm_flag_bytes(void) {
  return ((int64_t)2 * kCommMaxBlocks * kCommMaxWorld + kCommMaxBlocks) * (int64_t)sizeof(uint32_t);
}

static unsigned g_comm_spin_limit = kCommSpinLimit;
extern "C" void sglb200_comm_set_wait_probes(uint32_t probes) { g_comm_spin_limit = probes == 0 ? kCommSpinLimit : probes; }

extern "C" int sglb200_comm_status_clear(void) {
  const int zero = 0;
  SGLB_CUDA(cudaMemcpyToSymbol(g_comm_status, &zero, sizeof(int)));
  return SGLB200_OK;
}

extern "C" int sglb200_comm_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_comm_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

extern "C" int sglb200_reduce_gather(const void* stage, void* const* reduced_ptrs, void* const* flag_ptrs, void* out,
                                     int world, int rank, int64_t M, int64_t N, int dtype, int max_blocks,
                                     void* stream) {
  SGLB_REQUIRE(world >= 2 && world <= kCommMaxWorld && rank >= 0 && rank < world, "reduce_gather: world %d, rank %d",
               world, rank);
  SGLB_REQUIRE(M > 0 && N > 0 && N % 8 == 0, "reduce_gather: rows %lld, N %lld (N must be a multiple of 8)",
               (long long)M, (long long)N);
  const int64_t rows_own = sglb200_push_rows_per_owner(M, world);
  SGLB_REQUIRE(dtype == 0 || dtype == 1, "reduce_gather: dtype %d (0 bf16, 1 fp16)", dtype);
  SGLB_REQUIRE(stage && reduced_ptrs && flag_ptrs && out && aligned16(stage) && aligned16(out),
               "reduce_gather: null or unaligned pointer");
  CommPeers c{};
  c.spin_limit = g_comm_spin_limit;
  c.stage = static_cast<const uint16_t*>(stage);
  for (int i = 0; i < world; ++i) {
    SGLB_REQUIRE(reduced_ptrs[i] && flag_ptrs[i] && aligned16(reduced_ptrs[i]), "reduce_gather: peer %d buffers", i);
    c.reduced[i] = static_cast<uint16_t*>(reduced_ptrs[i]);
    c.flags[i] = static_cast<uint32_t*>(flag_ptrs[i]);
  }
  const int64_t chunks = rows_own * N / 8, total_chunks = M * N / 8;
  int64_t blocks = (chunks + kCommThreads - 1) / kCommThreads;
  const int sms = sm_count();
  if (blocks > sms) blocks = sms;
  if (blocks > kCommMaxBlocks) blocks = kCommMaxBlocks;
  if (max_blocks > 0 && blocks > max_blocks) blocks = max_blocks;  // (the same on every rank: block b pairs with block b)
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    reduce_gather_kernel<false><<<(unsigned)blocks, kCommThreads, 0, st>>>(c, static_cast<uint16_t*>(out), chunks,
                                                                           total_chunks, world, rank);
  else
    reduce_gather_kernel<true><<<(unsigned)blocks, kCommThreads, 0, st>>>(c, static_cast<uint16_t*>(out), chunks,
                                                                          total_chunks, world, rank);
  SGLB_CUDA(cudaGetLastError());
  return SGLB200_OK;
}
