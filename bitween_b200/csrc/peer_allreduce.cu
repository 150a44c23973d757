// All-reduce of the row-parallel layers' partial outputs over peer memory (NVLink / NVSwitch),
// without NCCL: every rank's quantized matmul writes its partial sums [M, N] fp16 straight into a
// buffer that the other GPUs of the node have mapped (CUDA IPC), and ONE kernel per rank then
//   1. tells every peer "my partial is complete" (a release store, system scope, into the
//      peer's flag array) and waits -- bounded -- for the same word from every peer,
//   2. adds the partials of all ranks in rank order (fp32 sums of the fp16 values, so every
//      rank produces the same bits) with 16-byte loads straight from the peers' memory,
//   3. writes the fp16 result into local memory.
// A decode step's all-reduce is 1 MiB: bound by latency, not bandwidth.  This kernel's latency
// is one flag round trip plus one pass of peer loads.
//
// Reuse of a buffer: callers alternate between two buffers; a rank can only enter call c+1's
// barrier after its own call c has completed, so when the barrier of call c+1 passes every
// peer has finished READING the buffer of call c-1, which call c+1 overwrites.
// Flags carry the call number (epoch), kept in device memory and advanced by the last block to
// finish, so that a captured CUDA graph replays correctly; nothing is ever reset.
// No multicast objects, no multimem instructions: plain peer loads and stores.
#include "bw_common.cuh"

namespace bw {
namespace {

constexpr int PEER_MAX_RANKS = 8;
constexpr int PEER_BLOCKS = 128;                // every rank launches the same grid: a flag slot per block and rank
constexpr int PEER_THREADS = 512;               // 64 K threads: one 16-byte chunk each for a 1 MiB all-reduce, a single round of peer loads
constexpr unsigned PEER_WAIT_LIMIT = 1u << 23;  // polls of >= 20 ns each: gives up after ~0.2-1 s

__device__ int g_peer_status = 0;

struct PeerArgs {
    const __half *buf[PEER_MAX_RANKS];   // rank r's partial sums (peer mappings; buf[rank] is local)
    unsigned *flag[PEER_MAX_RANKS];      // rank r's flag array [2 phases][PEER_BLOCKS][PEER_MAX_RANKS]
    __half *res[PEER_MAX_RANKS];         // two-shot form: rank r's reduced slice (peer mappings; res[rank] is local)
};

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// state[0] = calls completed (epoch), state[1] = blocks of the running call that have finished
__global__ void __launch_bounds__(PEER_THREADS) peer_allreduce_kernel(const PeerArgs a, int rank, int world, __half *__restrict__ out,
                                                             int64_t chunks, unsigned *__restrict__ state) {
    __shared__ int timed_out;
    const unsigned epoch = *reinterpret_cast<volatile unsigned *>(state) + 1u;
    if (threadIdx.x == 0) timed_out = 0;
    __syncthreads();
    if (threadIdx.x < world && threadIdx.x != rank) {
        const int peer = threadIdx.x;
        // my partial (written by the kernel before this one in the stream) is complete
        st_release_sys(a.flag[peer] + blockIdx.x * PEER_MAX_RANKS + rank, epoch);
        const unsigned *mine = a.flag[rank] + blockIdx.x * PEER_MAX_RANKS + peer;
        unsigned tries = 0;
        while (ld_acquire_sys(mine) != epoch) {
            __nanosleep(20);
            if (++tries > PEER_WAIT_LIMIT) {
                timed_out = 1;
                atomicExch(&g_peer_status, 1);
                break;
            }
        }
    }
    __syncthreads();
    if (!timed_out) {
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (int64_t)gridDim.x * blockDim.x) {
            // all ranks' chunks are requested before the first is used (one peer round trip, not `world`);
            // L1 is not coherent with the peers' writes and the addresses repeat call after call: bypass it
            uint4 v[PEER_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < PEER_MAX_RANKS; ++r)
                if (r < world) v[r] = __ldcg(reinterpret_cast<const uint4 *>(a.buf[r]) + i);
            float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int r = 0; r < PEER_MAX_RANKS; ++r) {
                if (r < world) {
                    const __half2 *h = reinterpret_cast<const __half2 *>(&v[r]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(h[j]);
                        acc[2 * j] += f.x;
                        acc[2 * j + 1] += f.y;
                    }
                }
            }
            uint4 o;
            __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
            reinterpret_cast<uint4 *>(out)[i] = o;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // the last block to finish advances the epoch (every block has read it by then)
        if (atomicAdd(state + 1, 1u) == gridDim.x - 1) {
            state[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned *>(state) = epoch;
        }
    }
}

// One block's barrier with the same block of every other rank: tell each peer (release, system
// scope), then wait -- bounded -- for each peer's word.  Called by all threads of the block.
__device__ __forceinline__ bool block_barrier(const PeerArgs &a, int rank, int world, int phase, unsigned epoch, int *timed_out) {
    __syncthreads();                                   // this block's writes so far come before the release below
    if (threadIdx.x < world && threadIdx.x != rank) {
        const int peer = threadIdx.x;
        const int slot = (phase * PEER_BLOCKS + blockIdx.x) * PEER_MAX_RANKS;
        st_release_sys(a.flag[peer] + slot + rank, epoch);
        const unsigned *mine = a.flag[rank] + slot + peer;
        unsigned tries = 0;
        while (ld_acquire_sys(mine) != epoch) {
            __nanosleep(20);
            if (++tries > PEER_WAIT_LIMIT) {
                *timed_out = 1;
                atomicExch(&g_peer_status, 1);
                break;
            }
        }
    }
    __syncthreads();
    return *timed_out == 0;
}

// Two-shot form for many ranks: every rank sums ONE slice of the data (reading that slice from every
// peer), publishes it in its own result buffer, and after a second barrier every rank collects the
// slices: (world-1)/world of the data is read twice instead of (world-1) times once.  Chunk j of a
// slice is always handled by the same block index on every rank, so the per-block barrier is enough.
__global__ void __launch_bounds__(PEER_THREADS) peer_allreduce2_kernel(const PeerArgs a, int rank, int world, __half *__restrict__ out,
                                                                       int64_t chunks, unsigned *__restrict__ state) {
    __shared__ int timed_out;
    const unsigned epoch = *reinterpret_cast<volatile unsigned *>(state) + 1u;
    if (threadIdx.x == 0) timed_out = 0;
    const int64_t per = (chunks + world - 1) / world;            // chunks per slice
    const int64_t stride = (int64_t)gridDim.x * blockDim.x, first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    bool ok = block_barrier(a, rank, world, 0, epoch, &timed_out);
    if (ok) {
        const int64_t lo = rank * per, n = min(per, chunks - lo);
        auto reduce_chunk = [&](const uint4 (&v)[PEER_MAX_RANKS]) {
            float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int r = 0; r < PEER_MAX_RANKS; ++r) {
                if (r < world) {
                    const __half2 *h = reinterpret_cast<const __half2 *>(&v[r]);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 f = __half22float2(h[q]);
                        acc[2 * q] += f.x;
                        acc[2 * q + 1] += f.y;
                    }
                }
            }
            uint4 o;
            __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
            for (int q = 0; q < 4; ++q) oh[q] = __floats2half2_rn(acc[2 * q], acc[2 * q + 1]);
            return o;
        };
        int64_t j = first;
        // two chunks per thread in flight (large messages are bound by the bytes in flight over NVLink)
        for (; j + stride < n; j += 2 * stride) {
            uint4 v0[PEER_MAX_RANKS], v1[PEER_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < PEER_MAX_RANKS; ++r)
                if (r < world) {
                    v0[r] = __ldcg(reinterpret_cast<const uint4 *>(a.buf[r]) + lo + j);
                    v1[r] = __ldcg(reinterpret_cast<const uint4 *>(a.buf[r]) + lo + j + stride);
                }
            const uint4 o0 = reduce_chunk(v0), o1 = reduce_chunk(v1);
            reinterpret_cast<uint4 *>(a.res[rank])[j] = o0;          // my slice, where the peers will fetch it
            reinterpret_cast<uint4 *>(a.res[rank])[j + stride] = o1;
            reinterpret_cast<uint4 *>(out)[lo + j] = o0;
            reinterpret_cast<uint4 *>(out)[lo + j + stride] = o1;
        }
        for (; j < n; j += stride) {
            uint4 v[PEER_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < PEER_MAX_RANKS; ++r)
                if (r < world) v[r] = __ldcg(reinterpret_cast<const uint4 *>(a.buf[r]) + lo + j);
            const uint4 o = reduce_chunk(v);
            reinterpret_cast<uint4 *>(a.res[rank])[j] = o;
            reinterpret_cast<uint4 *>(out)[lo + j] = o;
        }
        ok = block_barrier(a, rank, world, 1, epoch, &timed_out);
    }
    if (ok) {
        for (int p = 0; p < world; ++p) {
            if (p == rank) continue;
            const int64_t lo = p * per, n = min(per, chunks - lo);
            int64_t j = first;
            for (; j + 3 * stride < n; j += 4 * stride) {            // four loads in flight per thread
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = __ldcg(reinterpret_cast<const uint4 *>(a.res[p]) + j + u * stride);
#pragma unroll
                for (int u = 0; u < 4; ++u) reinterpret_cast<uint4 *>(out)[lo + j + u * stride] = v[u];
            }
            for (; j < n; j += stride)
                reinterpret_cast<uint4 *>(out)[lo + j] = __ldcg(reinterpret_cast<const uint4 *>(a.res[p]) + j);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(state + 1, 1u) == gridDim.x - 1) {
            state[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned *>(state) = epoch;
        }
    }
}

}  // namespace

size_t peer_flag_bytes() { return (size_t)2 * PEER_BLOCKS * PEER_MAX_RANKS * sizeof(unsigned); }
size_t peer_state_bytes() { return 2 * sizeof(unsigned); }

int peer_device_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_peer_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) (void)cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int));
    return v;
}

// bufs / res / flags: host arrays of `world` device pointers (this process's mappings of every rank's buffers).
// res == nullptr: one-shot form (every rank reads everything); else the two-shot form through the result buffers.
int peer_allreduce_f16(const void *const *bufs, void *const *res, void *const *flags, int rank, int world, void *out, int64_t count,
                       void *state, cudaStream_t st) {
    if (world < 1 || world > PEER_MAX_RANKS || rank < 0 || rank >= world) return BW_ERR_SHAPE;
    if (count < 0 || count % 8 != 0) return BW_ERR_SHAPE;       // whole 16-byte chunks
    if (count == 0) return BW_OK;
    if (!out || !state || !bufs || !flags) return BW_ERR_NULL;
    PeerArgs a = {};
    for (int r = 0; r < world; ++r) {
        if (!bufs[r] || !flags[r] || (res && !res[r])) return BW_ERR_NULL;
        if (!aligned_to(bufs[r], 16) || !aligned_to(flags[r], 4) || (res && !aligned_to(res[r], 16))) return BW_ERR_ALIGN;
        a.buf[r] = reinterpret_cast<const __half *>(bufs[r]);
        a.flag[r] = reinterpret_cast<unsigned *>(flags[r]);
        a.res[r] = res ? reinterpret_cast<__half *>(res[r]) : nullptr;
    }
    if (!aligned_to(out, 16)) return BW_ERR_ALIGN;
    if (res) {
        peer_allreduce2_kernel<<<PEER_BLOCKS, PEER_THREADS, 0, st>>>(a, rank, world, reinterpret_cast<__half *>(out), count / 8,
                                                                     reinterpret_cast<unsigned *>(state));
        return check_launch("peer_allreduce2_kernel");
    }
    peer_allreduce_kernel<<<PEER_BLOCKS, PEER_THREADS, 0, st>>>(a, rank, world, reinterpret_cast<__half *>(out), count / 8,
                                                               reinterpret_cast<unsigned *>(state));
    return check_launch("peer_allreduce_kernel");
}

}  // namespace bw
