// All-to-all of equal blocks written straight into the destination ranks' memory.
//
// Every rank holds a receive buffer that its peers have mapped into their own address space
// (symmetric memory: plain peer mappings over NVLink, no multicast).  Block t of this rank's send
// buffer goes to slot `rank` of rank t's receive buffer, so one launch on every rank is the whole
// exchange: 16-byte loads from local memory, 16-byte stores to local or peer memory, all SMs.  The
// caller orders it against the consumers with the cross-rank barrier below (b200pf_peer_barrier);
// the copy kernels themselves never wait on another GPU.
#include "common.cuh"

namespace b200pf {

constexpr int PEER_MAX_RANKS = 16;
struct PeerPtrs {
    unsigned long long recv[PEER_MAX_RANKS];     // receive buffer of rank t as mapped on this device
};

// Cross-rank barrier on symmetric signal pads (one 32-bit slot per sender in every rank's pad), run by one warp.
// Lane t tells rank t "rank `rank` has reached generation `gen`" with a system-scope release store into slot
// `rank` of rank t's pad, then waits until slot t of its own pad shows that rank t has reached `gen` too.
// Generations only grow, and a rank can be at most one barrier ahead of a peer that is still waiting, so the
// test is "slot - gen >= 0" in wrap-around arithmetic.  After an exchange on the same stream it tells the
// receivers that this rank's blocks have landed and holds this rank's consumers back until every sender's have.
// The wait is bounded: after `limit_ns` without the peer's signal the lane ORs DEV_STATUS_PEER_TIMEOUT into the
// device status word and returns.  Nothing traps; the context stays usable and the host reads the word.
struct BarrierArgs {
    PeerPtrs pads;
    unsigned int gen;
    int rank, world;         // world 0: no barrier
    int channel;
    unsigned long long limit_ns;
    unsigned int* status;
};
__device__ __forceinline__ void peer_barrier_lane(const BarrierArgs& b, int t) {
    if (t >= b.world) return;
    __threadfence_system();
    unsigned int* remote = reinterpret_cast<unsigned int*>(b.pads.recv[t]) + b.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(b.gen) : "memory");
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(b.pads.recv[b.rank]) + t;
    unsigned long long t0 = 0;
    for (unsigned int spins = 0;; ++spins) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int)(v - b.gen) >= 0) return;
        if ((spins & 63u) == 63u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            if (now - t0 > b.limit_ns) {
                atomicOr(b.status, DEV_STATUS_PEER_TIMEOUT);
                return;
            }
            __nanosleep(200);
        }
    }
}
__global__ void __launch_bounds__(32) peer_barrier_kernel(BarrierArgs b) { peer_barrier_lane(b, threadIdx.x); }

// Tail of an exchange kernel that carries its own barrier (b.world > 0): every CTA makes its stores visible
// system-wide (one fence by thread 0 behind a CTA barrier: a fence per thread cost more than the copy gained from
// short CTAs) and counts itself in; the CTA that completes the count resets it for the next launch and runs
// the barrier, so the kernel ends when every peer's blocks have landed here.  One launch instead of two.
constexpr int PEER_CHANNELS = 8;      // exchanges that may run at the same time on one device use different channels
__device__ unsigned int g_exchange_ctas_done[PEER_CHANNELS];
__device__ __forceinline__ void exchange_tail(const BarrierArgs& b) {
    if (b.world <= 0) return;
    __shared__ unsigned int is_last;
    __syncthreads();                          // the CTA's stores are ordered before thread 0's fence ...
    if (threadIdx.x == 0) {
        __threadfence_system();               // ... which makes them visible system-wide before the count goes up
        const unsigned int done = atomicAdd(&g_exchange_ctas_done[b.channel], 1u);
        is_last = (done == gridDim.x - 1);
        if (is_last) g_exchange_ctas_done[b.channel] = 0;   // the next launch on this channel starts after this one has ended
    }
    __syncthreads();
    if (is_last && threadIdx.x < 32) peer_barrier_lane(b, threadIdx.x);
}

// Each thread moves UNROLL independent 16-byte pieces per step (all loads first, then all stores): NVLink stores
// are posted, so what limits the rate is how many bytes a thread has in flight between its loads and stores.
constexpr int PEER_UNROLL = 4;
// Grid cap in CTAs per SM (8 x 256 threads are resident at once).  Alone between two GPUs more and shorter CTAs copy
// faster (64 MB each way plus 64 MB local: 8 per SM 571 GB/s per direction, 16: 616, 64: 646), but inside the trunk,
// with the barrier tail and the single track's kernels on the side stream, 64 per SM made a block 5 % slower than
// 8 or 16 (4.85 vs 4.60 ms at 2 GPUs), which measured the same.
constexpr int PEER_CTAS_PER_SM = 16;

__global__ void __launch_bounds__(256)
peer_scatter_kernel(const uint4* __restrict__ send, PeerPtrs peers, long long block_vec, int rank, int world, BarrierArgs bar) {
    const long long total = block_vec * world;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (PEER_UNROLL - 1) * stride < total; i += PEER_UNROLL * stride) {
        uint4 v[PEER_UNROLL];
        uint4* dst[PEER_UNROLL];
#pragma unroll
        for (int u = 0; u < PEER_UNROLL; ++u) {
            // start every rank on a different destination so that no receiver is hit by all senders at once
            const long long e = i + u * stride, slot = e / block_vec, off = e - slot * block_vec;
            const int t = (int)((slot + rank) % world);
            dst[u] = reinterpret_cast<uint4*>(peers.recv[t]) + (long long)rank * block_vec + off;
            v[u] = __ldg(send + (long long)t * block_vec + off);
        }
#pragma unroll
        for (int u = 0; u < PEER_UNROLL; ++u) *dst[u] = v[u];
    }
    for (; i < total; i += stride) {
        const long long slot = i / block_vec, off = i - slot * block_vec;
        const int t = (int)((slot + rank) % world);
        uint4* d = reinterpret_cast<uint4*>(peers.recv[t]) + (long long)rank * block_vec + off;
        *d = __ldg(send + (long long)t * block_vec + off);
    }
    exchange_tail(bar);
}

// All-to-all of blocks that are not contiguous on one or both sides: block t consists of `chunks` pieces of
// chunk_vec 16-byte vectors; piece q is read at send + t * src_block + q * src_chunk and written to rank t at
// recv[t] + rank * dst_slot + q * dst_chunk (all in vectors).  This is the row-shard <-> column-shard transposition
// of the pair tensor without a packing copy on either side.
struct StridedCopy {
    unsigned int chunks, chunk_vec;
    long long src_block, src_chunk, dst_slot, dst_chunk;
};
__global__ void __launch_bounds__(256)
peer_scatter_strided_kernel(const uint4* __restrict__ send, PeerPtrs peers, StridedCopy c, int rank, int world, BarrierArgs bar) {
    const unsigned int block_vec = c.chunks * c.chunk_vec;
    const unsigned long long total = (unsigned long long)block_vec * world;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i < total; i += PEER_UNROLL * stride) {
        uint4 v[PEER_UNROLL];
        uint4* dst[PEER_UNROLL];
#pragma unroll
        for (int u = 0; u < PEER_UNROLL; ++u) {
            const unsigned long long e = i + u * stride;
            dst[u] = nullptr;
            if (e < total) {
                const unsigned int slot = (unsigned int)(e / block_vec), rem = (unsigned int)(e - (unsigned long long)slot * block_vec);
                const unsigned int q = rem / c.chunk_vec, off = rem - q * c.chunk_vec;
                const int t = (int)((slot + rank) % world);
                dst[u] = reinterpret_cast<uint4*>(peers.recv[t]) + rank * c.dst_slot + q * c.dst_chunk + off;
                v[u] = __ldg(send + t * c.src_block + q * c.src_chunk + off);
            }
        }
#pragma unroll
        for (int u = 0; u < PEER_UNROLL; ++u)
            if (dst[u]) *dst[u] = v[u];
    }
    exchange_tail(bar);
}

// The same strided all-to-all with the elements narrowed on the way: fp32 in this rank's memory, bf16 on the wire
// and in the receivers' buffers.  All StridedCopy fields count DESTINATION vectors (8 bf16 = 16 bytes); a source
// vector is the matching 8 floats (two 16-byte loads).
__global__ void __launch_bounds__(256)
peer_scatter_strided_f32_bf16_kernel(const float4* __restrict__ send, PeerPtrs peers, StridedCopy c, int rank, int world, BarrierArgs bar) {
    const unsigned int block_vec = c.chunks * c.chunk_vec;
    const unsigned long long total = (unsigned long long)block_vec * world;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i < total; i += PEER_UNROLL * stride) {
        float4 v[PEER_UNROLL][2];
        uint4* dst[PEER_UNROLL];
#pragma unroll
        for (int u = 0; u < PEER_UNROLL; ++u) {
            const unsigned long long e = i + u * stride;
            dst[u] = nullptr;
            if (e < total) {
                const unsigned int slot = (unsigned int)(e / block_vec), rem = (unsigned int)(e - (unsigned long long)slot * block_vec);
                const unsigned int q = rem / c.chunk_vec, off = rem - q * c.chunk_vec;
                const int t = (int)((slot + rank) % world);
                dst[u] = reinterpret_cast<uint4*>(peers.recv[t]) + rank * c.dst_slot + q * c.dst_chunk + off;
                const float4* src = send + 2 * (t * c.src_block + q * c.src_chunk + off);
                v[u][0] = __ldg(src);
                v[u][1] = __ldg(src + 1);
            }
        }
#pragma unroll
        for (int u = 0; u < PEER_UNROLL; ++u)
            if (dst[u]) *dst[u] = make_uint4(pack_bf16x2(v[u][0].x, v[u][0].y), pack_bf16x2(v[u][0].z, v[u][0].w),
                                             pack_bf16x2(v[u][1].x, v[u][1].y), pack_bf16x2(v[u][1].z, v[u][1].w));
    }
    exchange_tail(bar);
}

// z += update (bf16 -> fp32), element-wise: how an update that crossed the wire in bf16 reaches the fp32 residual stream.
__global__ void __launch_bounds__(256) add_bf16_kernel(float4* __restrict__ z, const uint2* __restrict__ upd, long long vec4) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vec4; i += stride) {
        const uint2 u = __ldg(upd + i);
        float4 v = z[i];
        v.x += bf16_lo(u.x); v.y += bf16_hi(u.x); v.z += bf16_lo(u.y); v.w += bf16_hi(u.y);
        z[i] = v;
    }
}

// All-gather form: the one block of this rank goes to slot `rank` of every rank's receive buffer.
__global__ void __launch_bounds__(256)
peer_broadcast_kernel(const uint4* __restrict__ send, PeerPtrs peers, long long block_vec, int rank, int world, BarrierArgs bar) {
    const long long total = block_vec * world;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long slot = i / block_vec, off = i - slot * block_vec;
        const int t = (int)((slot + rank) % world);
        uint4* dst = reinterpret_cast<uint4*>(peers.recv[t]) + (long long)rank * block_vec + off;
        *dst = __ldg(send + off);
    }
    exchange_tail(bar);
}

}  // namespace b200pf

using namespace b200pf;

static int fill_barrier(BarrierArgs* b, const b200pf_peer_sync* sync, int rank, int world, const char* who) {
    *b = BarrierArgs{};
    if (!sync) return B200PF_OK;
    B200PF_REQUIRE(sync->pad_ptrs && sync->timeout_ns > 0 && sync->channel >= 0 && sync->channel < PEER_CHANNELS, B200PF_ERR_INVALID,
                   "%s: the barrier needs signal pads, a positive limit and a channel below %d", who, PEER_CHANNELS);
    for (int t = 0; t < world; ++t) {
        B200PF_REQUIRE(sync->pad_ptrs[t] != 0 && sync->pad_ptrs[t] % 4 == 0, B200PF_ERR_INVALID, "%s: bad signal pad of rank %d", who, t);
        b->pads.recv[t] = sync->pad_ptrs[t];
    }
    b->gen = sync->generation; b->rank = rank; b->world = world; b->channel = sync->channel;
    b->limit_ns = (unsigned long long)sync->timeout_ns;
    b->status = device_status_word();
    B200PF_REQUIRE(b->status, B200PF_ERR_CUDA, "%s: no device status word", who);
    return B200PF_OK;
}

extern "C" int b200pf_peer_barrier(const unsigned long long* pad_ptrs, unsigned int generation, int rank, int world,
                                   long long timeout_ns, void* stream) {
    B200PF_REQUIRE(pad_ptrs && world > 0 && world <= PEER_MAX_RANKS && rank >= 0 && rank < world, B200PF_ERR_INVALID,
                   "peer_barrier: bad argument (at most %d ranks)", PEER_MAX_RANKS);
    B200PF_REQUIRE(timeout_ns > 0, B200PF_ERR_INVALID, "peer_barrier: the wait must have a positive limit");
    b200pf_peer_sync sync{pad_ptrs, generation, timeout_ns, 0};
    BarrierArgs b;
    int rc = fill_barrier(&b, &sync, rank, world, "peer_barrier");
    if (rc != B200PF_OK) return rc;
    peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(b);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

static int peer_launch(bool broadcast, const void* send, const unsigned long long* recv_ptrs, long long block_bytes,
                       int rank, int world, const b200pf_peer_sync* sync, void* stream) {
    B200PF_REQUIRE(send && recv_ptrs && world > 0 && world <= PEER_MAX_RANKS && rank >= 0 && rank < world, B200PF_ERR_INVALID,
                   "peer_scatter: bad argument (at most %d ranks)", PEER_MAX_RANKS);
    B200PF_REQUIRE(block_bytes > 0 && block_bytes % 16 == 0 && aligned16(send), B200PF_ERR_INVALID,
                   "peer_scatter: blocks must be 16-byte multiples and 16-byte aligned");
    PeerPtrs p{};
    for (int t = 0; t < world; ++t) {
        B200PF_REQUIRE(recv_ptrs[t] != 0 && recv_ptrs[t] % 16 == 0, B200PF_ERR_INVALID, "peer_scatter: bad receive pointer of rank %d", t);
        p.recv[t] = recv_ptrs[t];
    }
    BarrierArgs bar;
    int rc = fill_barrier(&bar, sync, rank, world, "peer_scatter");
    if (rc != B200PF_OK) return rc;
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long vec = block_bytes / 16;
    long long blocks = (vec * world + 255) / 256;
    if (blocks > (long long)sms * PEER_CTAS_PER_SM) blocks = (long long)sms * PEER_CTAS_PER_SM;
    if (broadcast)
        peer_broadcast_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(static_cast<const uint4*>(send), p, vec, rank, world, bar);
    else
        peer_scatter_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(static_cast<const uint4*>(send), p, vec, rank, world, bar);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

static int strided_launch(const void* send, const unsigned long long* recv_ptrs, long long chunk_bytes, int chunks,
                          long long src_block_stride, long long src_chunk_stride, long long dst_slot_stride, long long dst_chunk_stride,
                          int rank, int world, const b200pf_peer_sync* sync, void* stream) {
    B200PF_REQUIRE(send && recv_ptrs && world > 0 && world <= PEER_MAX_RANKS && rank >= 0 && rank < world, B200PF_ERR_INVALID,
                   "peer_scatter_strided: bad argument (at most %d ranks)", PEER_MAX_RANKS);
    B200PF_REQUIRE(chunks > 0 && chunk_bytes > 0 && chunk_bytes % 16 == 0 && aligned16(send) && src_block_stride % 16 == 0 &&
                       src_chunk_stride % 16 == 0 && dst_slot_stride % 16 == 0 && dst_chunk_stride % 16 == 0 &&
                       src_block_stride >= 0 && src_chunk_stride >= chunk_bytes && dst_slot_stride >= 0 && dst_chunk_stride >= chunk_bytes,
                   B200PF_ERR_INVALID, "peer_scatter_strided: sizes and strides must be non-negative 16-byte multiples, chunk strides >= the chunk");
    B200PF_REQUIRE(chunk_bytes / 16 < (1ll << 31) && (long long)chunks * (chunk_bytes / 16) < (1ll << 32), B200PF_ERR_UNSUPPORTED,
                   "peer_scatter_strided: block too large");
    PeerPtrs p{};
    for (int t = 0; t < world; ++t) {
        B200PF_REQUIRE(recv_ptrs[t] != 0 && recv_ptrs[t] % 16 == 0, B200PF_ERR_INVALID, "peer_scatter_strided: bad receive pointer of rank %d", t);
        p.recv[t] = recv_ptrs[t];
    }
    BarrierArgs bar;
    int rc = fill_barrier(&bar, sync, rank, world, "peer_scatter_strided");
    if (rc != B200PF_OK) return rc;
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    StridedCopy c{(unsigned int)chunks, (unsigned int)(chunk_bytes / 16), src_block_stride / 16, src_chunk_stride / 16,
                  dst_slot_stride / 16, dst_chunk_stride / 16};
    const long long vec = (long long)chunks * (chunk_bytes / 16) * world;
    long long blocks = (vec + 256 * PEER_UNROLL - 1) / (256 * PEER_UNROLL);
    if (blocks > (long long)sms * PEER_CTAS_PER_SM) blocks = (long long)sms * PEER_CTAS_PER_SM;
    peer_scatter_strided_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(static_cast<const uint4*>(send), p, c, rank, world, bar);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_peer_scatter_strided_f32_bf16_sync(const float* send, const unsigned long long* recv_ptrs, long long chunk_elems, int chunks,
                                                         long long src_block_stride, long long src_chunk_stride,
                                                         long long dst_slot_stride, long long dst_chunk_stride, int rank, int world,
                                                         const b200pf_peer_sync* sync, void* stream) {
    B200PF_REQUIRE(send && recv_ptrs && sync && world > 0 && world <= PEER_MAX_RANKS && rank >= 0 && rank < world, B200PF_ERR_INVALID,
                   "peer_scatter_strided_f32_bf16: bad argument (at most %d ranks)", PEER_MAX_RANKS);
    B200PF_REQUIRE(chunks > 0 && chunk_elems > 0 && chunk_elems % 8 == 0 && (reinterpret_cast<uintptr_t>(send) & 31) == 0 &&
                       src_block_stride % 8 == 0 && src_chunk_stride % 8 == 0 && dst_slot_stride % 8 == 0 && dst_chunk_stride % 8 == 0 &&
                       src_block_stride >= 0 && src_chunk_stride >= chunk_elems && dst_slot_stride >= 0 && dst_chunk_stride >= chunk_elems,
                   B200PF_ERR_INVALID, "peer_scatter_strided_f32_bf16: sizes and strides count elements, multiples of 8, chunk strides >= the chunk; "
                                       "the source must be 32-byte aligned");
    B200PF_REQUIRE(chunk_elems / 8 < (1ll << 31) && (long long)chunks * (chunk_elems / 8) < (1ll << 32), B200PF_ERR_UNSUPPORTED,
                   "peer_scatter_strided_f32_bf16: block too large");
    PeerPtrs p{};
    for (int t = 0; t < world; ++t) {
        B200PF_REQUIRE(recv_ptrs[t] != 0 && recv_ptrs[t] % 16 == 0, B200PF_ERR_INVALID, "peer_scatter_strided_f32_bf16: bad receive pointer of rank %d", t);
        p.recv[t] = recv_ptrs[t];
    }
    BarrierArgs bar;
    int rc = fill_barrier(&bar, sync, rank, world, "peer_scatter_strided_f32_bf16");
    if (rc != B200PF_OK) return rc;
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    StridedCopy c{(unsigned int)chunks, (unsigned int)(chunk_elems / 8), src_block_stride / 8, src_chunk_stride / 8,
                  dst_slot_stride / 8, dst_chunk_stride / 8};
    const long long vec = (long long)chunks * (chunk_elems / 8) * world;
    long long blocks = (vec + 256 * PEER_UNROLL - 1) / (256 * PEER_UNROLL);
    if (blocks > (long long)sms * PEER_CTAS_PER_SM) blocks = (long long)sms * PEER_CTAS_PER_SM;
    peer_scatter_strided_f32_bf16_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const float4*>(send), p, c, rank, world, bar);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_add_bf16(float* z, const b200pf_bf16* upd, long long n_elems, void* stream) {
    B200PF_REQUIRE(z && upd && n_elems > 0 && n_elems % 4 == 0 && aligned16(z) && (reinterpret_cast<uintptr_t>(upd) & 7) == 0,
                   B200PF_ERR_INVALID, "add_bf16: element count must be a multiple of 4, z 16-byte and the update 8-byte aligned");
    int dev = 0, sms = 148;
    B200PF_CUDA(cudaGetDevice(&dev));
    B200PF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long vec4 = n_elems / 4;
    long long blocks = (vec4 + 255) / 256;
    if (blocks > (long long)sms * 16) blocks = (long long)sms * 16;
    add_bf16_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<float4*>(z), reinterpret_cast<const uint2*>(upd), vec4);
    B200PF_LAUNCH_CHECK();
    return B200PF_OK;
}

extern "C" int b200pf_peer_scatter_strided(const void* send, const unsigned long long* recv_ptrs, long long chunk_bytes, int chunks,
                                           long long src_block_stride, long long src_chunk_stride,
                                           long long dst_slot_stride, long long dst_chunk_stride, int rank, int world, void* stream) {
    return strided_launch(send, recv_ptrs, chunk_bytes, chunks, src_block_stride, src_chunk_stride, dst_slot_stride, dst_chunk_stride,
                          rank, world, nullptr, stream);
}

extern "C" int b200pf_peer_scatter(const void* send, const unsigned long long* recv_ptrs, long long block_bytes,
                                   int rank, int world, void* stream) {
    return peer_launch(false, send, recv_ptrs, block_bytes, rank, world, nullptr, stream);
}

extern "C" int b200pf_peer_broadcast(const void* send, const unsigned long long* recv_ptrs, long long block_bytes,
                                     int rank, int world, void* stream) {
    return peer_launch(true, send, recv_ptrs, block_bytes, rank, world, nullptr, stream);
}

extern "C" int b200pf_peer_scatter_sync(const void* send, const unsigned long long* recv_ptrs, long long block_bytes,
                                        int rank, int world, const b200pf_peer_sync* sync, void* stream) {
    B200PF_REQUIRE(sync, B200PF_ERR_INVALID, "peer_scatter_sync: the barrier description is missing");
    return peer_launch(false, send, recv_ptrs, block_bytes, rank, world, sync, stream);
}

extern "C" int b200pf_peer_broadcast_sync(const void* send, const unsigned long long* recv_ptrs, long long block_bytes,
                                          int rank, int world, const b200pf_peer_sync* sync, void* stream) {
    B200PF_REQUIRE(sync, B200PF_ERR_INVALID, "peer_broadcast_sync: the barrier description is missing");
    return peer_launch(true, send, recv_ptrs, block_bytes, rank, world, sync, stream);
}

extern "C" int b200pf_peer_scatter_strided_sync(const void* send, const unsigned long long* recv_ptrs, long long chunk_bytes, int chunks,
                                                long long src_block_stride, long long src_chunk_stride,
                                                long long dst_slot_stride, long long dst_chunk_stride, int rank, int world,
                                                const b200pf_peer_sync* sync, void* stream) {
    B200PF_REQUIRE(sync, B200PF_ERR_INVALID, "peer_scatter_strided_sync: the barrier description is missing");
    return strided_launch(send, recv_ptrs, chunk_bytes, chunks, src_block_stride, src_chunk_stride, dst_slot_stride, dst_chunk_stride,
                          rank, world, sync, stream);
}
