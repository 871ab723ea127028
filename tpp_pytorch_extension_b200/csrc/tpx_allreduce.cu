// All-reduce (SUM) of a small bf16 tensor over the tensor-parallel ranks of one node, through peer memory.
//
// Replaces tpp_llm.allreduce after the row-parallel linears of the decoder block (src/csrc/llm/fused_llm_infer.cpp:101-119,
// :1263-1277), whose reference implementation is a shared-memory all-reduce between the ranks of one host
// (src/csrc/shm_coll.cpp) with fp32 accumulation of the bf16 inputs. The payload of a decode step is tokens x d_model
// bf16 (8 KiB .. 1 MiB): far below the size at which a library collective reaches NVLink bandwidth, so what counts is
// latency. One kernel per call on every rank, no host synchronisation:
//   1. every CTA copies its share of the input into this rank's exchange buffer (memory every peer can read),
//   2. tells the same CTA of every peer that the share is there (a release store of the call's epoch into the peer's
//      flag array) and waits for the peers' flags (bounded: a peer that never arrives ends the wait with an error code,
//      the kernel finishes and the host reads the code),
//   3. reads the share from every rank's buffer with plain peer loads over NVLink, adds in rank order in fp32 (every rank
//      gets bit-identical sums) and writes bf16.
// The exchange buffers are double buffered by call parity: a rank rewrites a buffer only two calls later, after the
// barrier of the call in between has shown that every peer finished reading it. The epoch lives in device memory and is
// advanced by the last CTA of each call, so a CUDA graph that recorded the call replays correctly.
#include "tpx_common.cuh"

namespace tpx {

constexpr int kArMaxRanks = 8;
constexpr int kArMaxCtas = 128;
constexpr int kArThreads = 512;
constexpr unsigned kArSpinLimit = 1u << 20;  // about a second of polling

struct ArParams {
  uint16_t* data;                       // in place: [n] bf16
  long long n;                          // elements, a multiple of 8
  uint16_t* buf[kArMaxRanks];           // every rank's exchange buffer (two halves of `half_elems` each)
  unsigned* flags[kArMaxRanks];         // every rank's flag array [kArMaxCtas][kArMaxRanks]
  unsigned* state;                      // this rank's: [0] epoch, [1] CTAs done, [2] error code
  long long half_elems;
  int rank, world;
};

__device__ __forceinline__ void ar_st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ar_ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ar_ld_peer(const void* p) {  // peer data: never from a stale cache line
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kArThreads) allreduce_bf16_kernel(ArParams p) {
  __shared__ unsigned s_epoch;
  pdl_trigger();
  pdl_wait();  // the input was written by the kernel before this one
  if (threadIdx.x == 0) s_epoch = ar_ld_acquire_sys(&p.state[0]) + 1u;  // this call's epoch (advanced by the last CTA of the call)
  __syncthreads();
  const unsigned epoch = s_epoch;
  const int cta = blockIdx.x, nctas = gridDim.x;
  const long long vecs = p.n / 8;                      // 16-byte vectors
  const long long v0 = vecs * cta / nctas, v1 = vecs * (cta + 1) / nctas;
  const long long half = (long long)(epoch & 1u) * p.half_elems;
  // 1. my share into my exchange buffer
  {
    const uint4* src = reinterpret_cast<const uint4*>(p.data);
    uint4* dst = reinterpret_cast<uint4*>(p.buf[p.rank] + half);
    for (long long i = v0 + threadIdx.x; i < v1; i += kArThreads) dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  // 2. flags: one thread per peer signals, then waits
  bool ok = true;
  if (threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    ar_st_release_sys(&p.flags[peer][cta * kArMaxRanks + p.rank], epoch);
    const unsigned* mine = &p.flags[p.rank][cta * kArMaxRanks + peer];
    unsigned spins = 0;
    while ((int)(ar_ld_acquire_sys(mine) - epoch) < 0) {
      if (++spins >= kArSpinLimit) { ok = false; break; }
      __nanosleep(40);
    }
    if (!ok) atomicExch(&p.state[2], 1u + (unsigned)peer);
  }
  __syncthreads();
  // 3. reduce my share over all ranks, in rank order
  {
    uint4* out = reinterpret_cast<uint4*>(p.data);
#pragma unroll 2
    for (long long i = v0 + threadIdx.x; i < v1; i += kArThreads) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] = 0.0f;
      uint4 v[kArMaxRanks];
#pragma unroll
      for (int r = 0; r < kArMaxRanks; r++)
        if (r < p.world) v[r] = ar_ld_peer(reinterpret_cast<const uint4*>(p.buf[r] + half) + i);
#pragma unroll
      for (int r = 0; r < kArMaxRanks; r++) {
        if (r < p.world) {
          const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
          for (int j = 0; j < 4; j++) {
            acc[2 * j] += bf16_bits_to_f32((uint16_t)(w[j] & 0xffff));
            acc[2 * j + 1] += bf16_bits_to_f32((uint16_t)(w[j] >> 16));
          }
        }
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; j++) o[j] = (uint32_t)f32_to_bf16_bits(acc[2 * j]) | ((uint32_t)f32_to_bf16_bits(acc[2 * j + 1]) << 16);
      out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  // the last CTA of the call advances the epoch for the next one
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned done = atomicAdd(&p.state[1], 1u);
    if (done == (unsigned)nctas - 1) {
      p.state[1] = 0;
      ar_st_release_sys(&p.state[0], epoch);
    }
  }
}

}  // namespace tpx

using namespace tpx;

extern "C" size_t tpx_allreduce_flag_bytes(void) { return (size_t)kArMaxCtas * kArMaxRanks * sizeof(unsigned); }

extern "C" int tpx_allreduce_bf16(uint16_t* data, int64_t n, int rank, int world, const uint64_t* buf_ptrs_host,
                                  const uint64_t* flag_ptrs_host, void* state, int64_t buf_elems, void* stream) {
  TPX_REQUIRE(data && buf_ptrs_host && flag_ptrs_host && state, TPX_ERR_ARG, "allreduce: null pointer");
  TPX_REQUIRE(world >= 2 && world <= kArMaxRanks && rank >= 0 && rank < world, TPX_ERR_ARG, "allreduce: %d ranks not supported (2..%d)", world,
              kArMaxRanks);
  TPX_REQUIRE(n > 0 && n % 8 == 0 && ((uintptr_t)data & 15) == 0, TPX_ERR_ARG, "allreduce: needs a 16-byte aligned tensor of a multiple of 8 elements");
  TPX_REQUIRE(buf_elems % 16 == 0 && n <= buf_elems / 2, TPX_ERR_SCRATCH, "allreduce: %ld elements do not fit half of the exchange buffer (%ld)",
              (long)n, (long)buf_elems);
  ArParams p = {};
  p.data = data; p.n = n; p.rank = rank; p.world = world; p.half_elems = buf_elems / 2;
  p.state = reinterpret_cast<unsigned*>(state);
  for (int r = 0; r < world; r++) {
    TPX_REQUIRE(buf_ptrs_host[r] && flag_ptrs_host[r], TPX_ERR_ARG, "allreduce: rank %d has no buffer", r);
    p.buf[r] = reinterpret_cast<uint16_t*>(buf_ptrs_host[r]);
    p.flags[r] = reinterpret_cast<unsigned*>(flag_ptrs_host[r]);
  }
  // enough CTAs to keep the NVLink loads of all peers in flight, few enough that every rank's grid is resident at once
  long long vecs = n / 8;
  int ctas = (int)((vecs + kArThreads * 2 - 1) / (kArThreads * 2));
  if (ctas < 1) ctas = 1;
  if (ctas > kArMaxCtas) ctas = kArMaxCtas;
  TPX_CUDA_OK(launch_pdl(allreduce_bf16_kernel, dim3((unsigned)ctas), dim3(kArThreads), 0, (cudaStream_t)stream, p));
  return TPX_OK;
}
