// Head <-> sequence re-sharding of [*, 128] bf16 rows between the GPUs of one node, written as
// stores into the peers' memory (NVLink through NVSwitch) instead of a library all-to-all.
//
//   push_heads: this rank's sequence shard x[n_loc, H, 128] is read once, contiguously, and row
//               (r, h) is stored into the buffer of the rank that owns head h, at
//               [slot(h), rank * n_loc + r, :] of its [H_r, N, 128] array.
//   push_seq:   this rank's head-sharded result y[H_r, N, 128] is read once, contiguously, and
//               row (i, n) is stored into rank n / n_loc at [n % n_loc, head(i), :] of its
//               [n_loc, H, 128] array.
//
// A row is 256 bytes: 16 lanes store one 128-bit word each, so every store instruction of a
// half-warp is one full NVLink write packet.  Neither kernel waits on another GPU: the caller
// orders "all stores landed" and "buffer may be overwritten" with stream-ordered collectives
// between the launches.  The reference runs on one GPU and has no counterpart of this file.
#include "common.cuh"

namespace svoo {

constexpr int kMaxPeers = 16;
constexpr int kMaxExchangeHeads = 128;

struct PeerTable {
  uint4* dst[kMaxPeers];             // destination array of every rank (peer-mapped device pointers)
  int16_t owner[kMaxExchangeHeads];  // push_heads: rank that owns head h      | push_seq: unused
  int16_t slot[kMaxExchangeHeads];   // push_heads: index of h within its rank | push_seq: head id of local index i
};

constexpr int kXchgUnroll = 4;

// rows = n_loc * H rows of x, flat index t = r * H + h.
__global__ void __launch_bounds__(256) push_heads_kernel(const uint4* __restrict__ x, const __grid_constant__ PeerTable tab,
                                                         int64_t rows, int H, int64_t n_loc, int64_t N, int rank) {
  const int lane = threadIdx.x % 16;
  const int64_t sub = (int64_t)blockIdx.x * 16 + threadIdx.x / 16;
  const int64_t stride = (int64_t)gridDim.x * 16;
  for (int64_t t0 = sub; t0 < rows; t0 += stride * kXchgUnroll) {
    uint4 v[kXchgUnroll];
#pragma unroll
    for (int u = 0; u < kXchgUnroll; ++u) {
      const int64_t t = t0 + u * stride;
      if (t < rows) v[u] = __ldcs(x + t * 16 + lane);
    }
#pragma unroll
    for (int u = 0; u < kXchgUnroll; ++u) {
      const int64_t t = t0 + u * stride;
      if (t < rows) {
        const int64_t r = t / H;
        const int h = (int)(t - r * H);
        uint4* d = tab.dst[tab.owner[h]];
        d[((int64_t)tab.slot[h] * N + (int64_t)rank * n_loc + r) * 16 + lane] = v[u];
      }
    }
  }
}

// rows = hr * N rows of y, flat index t = i * N + n.
__global__ void __launch_bounds__(256) push_seq_kernel(const uint4* __restrict__ y, const __grid_constant__ PeerTable tab,
                                                       int64_t rows, int H, int64_t n_loc, int64_t N) {
  const int lane = threadIdx.x % 16;
  const int64_t sub = (int64_t)blockIdx.x * 16 + threadIdx.x / 16;
  const int64_t stride = (int64_t)gridDim.x * 16;
  for (int64_t t0 = sub; t0 < rows; t0 += stride * kXchgUnroll) {
    uint4 v[kXchgUnroll];
#pragma unroll
    for (int u = 0; u < kXchgUnroll; ++u) {
      const int64_t t = t0 + u * stride;
      if (t < rows) v[u] = __ldcs(y + t * 16 + lane);
    }
#pragma unroll
    for (int u = 0; u < kXchgUnroll; ++u) {
      const int64_t t = t0 + u * stride;
      if (t < rows) {
        const int64_t i = t / N;
        const int64_t n = t - i * N;
        const int64_t p = n / n_loc;
        uint4* d = tab.dst[p];
        d[((n - p * n_loc) * H + tab.slot[i]) * 16 + lane] = v[u];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Barrier over the ranks of one node through flag words in peer-mapped memory: lane p stores this
// rank's epoch into rank p's flag array and then waits until rank p's epoch has arrived in its own.
// Launched after the kernels whose stores it publishes, on the same stream: a kernel's stores to
// peer memory are performed when it completes, the release store of the flag comes after that,
// and the acquire load on the other side orders the reader's later kernels behind it.
// Each rank runs this kernel on its own GPU.  The wait is bounded (~2 s of clock64); on expiry the
// status word is set and the kernel returns, so a missing rank cannot hang the others.
// ---------------------------------------------------------------------------------------------
struct PeerFlagTable {
  uint32_t* flags[kMaxPeers];
};
constexpr long long kBarrierCycles = 4000000000LL;

__global__ void peer_barrier_kernel(const __grid_constant__ PeerFlagTable tab, int rank, int world, int slot0,
                                    uint32_t epoch, int32_t* __restrict__ status) {
  const int p = threadIdx.x;
  if (p >= world) return;
  uint32_t* remote = tab.flags[p] + slot0 + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const uint32_t* mine = tab.flags[rank] + slot0 + p;
  const long long t0 = clock64();
  for (;;) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if ((int32_t)(seen - epoch) >= 0) break;             // epochs only grow; the difference is wrap-safe
    if (clock64() - t0 > kBarrierCycles) {
      atomicExch(status, 1);
      break;
    }
  }
}

cudaError_t launch_peer_barrier(void* const* peer_flags, int world, int rank, int slot0, uint32_t epoch, int32_t* status,
                                cudaStream_t st) {
  PeerFlagTable tab{};
  for (int p = 0; p < world; ++p) tab.flags[p] = (uint32_t*)peer_flags[p];
  peer_barrier_kernel<<<1, 32, 0, st>>>(tab, rank, world, slot0, epoch, status);
  count_launches(1);
  return cudaGetLastError();
}

static int exchange_grid() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms * 8;
}

cudaError_t launch_push_heads(const void* x, void* const* peer_dst, const int32_t* owner, const int32_t* slot, int world,
                              int rank, int64_t n_loc, int H, cudaStream_t st) {
  PeerTable tab{};
  for (int p = 0; p < world; ++p) tab.dst[p] = (uint4*)peer_dst[p];
  for (int h = 0; h < H; ++h) {
    tab.owner[h] = (int16_t)owner[h];
    tab.slot[h] = (int16_t)slot[h];
  }
  push_heads_kernel<<<exchange_grid(), 256, 0, st>>>((const uint4*)x, tab, n_loc * H, H, n_loc, n_loc * world, rank);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t launch_push_seq(const void* y, void* const* peer_dst, const int32_t* my_heads, int world, int64_t n_loc,
                            int H, int hr, cudaStream_t st) {
  PeerTable tab{};
  for (int p = 0; p < world; ++p) tab.dst[p] = (uint4*)peer_dst[p];
  for (int i = 0; i < hr; ++i) tab.slot[i] = (int16_t)my_heads[i];
  const int64_t N = n_loc * world;
  push_seq_kernel<<<exchange_grid(), 256, 0, st>>>((const uint4*)y, tab, (int64_t)hr * N, H, n_loc, N);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
