// All-reduce over peer memory for the row-parallel weight-only GEMM (one process per GPU, one node,
// NVLink 5 through NVSwitch). It takes the place of the ncclAllReduce that follows the plugin in the
// reference (cpp/tensorrt_llm/plugins/ncclPlugin/allreducePlugin.cpp:407) and follows the idea of the
// reference's own custom all-reduce for dense layers (one-shot and two-shot kernels,
// cpp/tensorrt_llm/kernels/customAllReduceKernels.cu:1307,1426; selection by message size,
// allreducePlugin.cpp:258-283), which the reference never applies to this path. Plain peer loads
// and stores only: no multicast objects, no cluster multicast.
//
// Every rank owns a workspace block that all ranks have mapped; every area below exists in two copies
// used by alternate calls. One kernel per call and rank. Three protocols:
//
//   Messages up to W4_ALLREDUCE_LL_MAX_BYTES travel as flagged packets: a 16-byte packet is
//   {data, call number, data, call number}, so a receiver that polls the packet sees data and flag
//   arrive together (each 8-byte half is written atomically). No fence, no separate flag, no barrier:
//   the latency of a step is one NVLink traversal. Twice the bytes cross the link, which does not
//   matter while latency dominates.
//     one-shot: every thread pushes its vectors of the local partial sums into the inbox of every peer,
//       then polls its own inbox for the same vectors of every peer and adds them in rank order in
//       fp32, so all ranks hold bit-identical results.
//     two-shot: the message is cut into one slice per rank. Rank j receives slice j from everybody,
//       adds the world copies (rank order, fp32, + bias), writes its own output and pushes the rounded
//       result to every peer's second inbox, where the peers poll for it. Each rank sends 2 * bytes
//       instead of (world - 1) * bytes.
//     In W4_ALLREDUCE_GATHER_ONLY mode the one-shot pushes are skipped: the decode GEMM in front has
//     already sent this rank's results as packets from its epilogue (w4_gemm_launch_push).
//   Larger messages (bandwidth-bound) use the two-shot scheme with plain data and per-chunk arrival
//   flags: push slices (system fence, release store of the call number into flag (sender, chunk) at
//   the owner), reduce, publish in the owner's `reduced` buffer (second flag set), pull. These use
//   areas of their own, so a packet poll can never meet plain data.
//
// Call numbers live in DEVICE memory (control word 0), not in a launch argument: every CTA reads the
// number at start, the last CTA to finish advances it. A captured CUDA graph can therefore be replayed
// any number of times, and the copy a call uses follows from the number's parity. Why two copies are
// enough: a rank can only start call e + 2 after every peer has taken part in call e + 1, which a peer
// does after its call e (and all its reads of copy e & 1) has finished. A packet left from an earlier
// call carries an older number and is never taken for a new one (numbers repeat after 2^32 calls).
//
// Nobody waits before having pushed everything it owes, and a thread only ever waits for peers, never
// for another CTA of its own launch; grids are at most kMaxCtas <= SM count, so all CTAs are resident.
// Waits are bounded in time: when one expires the kernel records W4_ERR_DEVICE_TIMEOUT in the device
// status word, skips the rest and returns (a peer that never arrives must not hang this GPU); `out` is
// then undefined and the workspace must be cleared on all ranks before it is used again.
#include "w4_common.cuh"
#include "w4_internal.h"

namespace w4
{
namespace ar
{

constexpr int kMaxRanks = W4_MAX_RANKS;
constexpr int kThreads = 512;       // flag protocol
constexpr int kPacketThreads = 128; // packet protocols
constexpr int kMaxCtas = W4_ALLREDUCE_MAX_CTAS; // chunks per message or slice
constexpr size_t kCtrlBytes = 256;
constexpr size_t kFlagBytes = size_t(2) * kMaxRanks * kMaxCtas * sizeof(uint32_t);
constexpr size_t kHeaderBytes = kCtrlBytes + 2 * kFlagBytes; // control, flags, flags2
constexpr size_t kOneShotMax = W4_ONESHOT_MAX_BYTES;
constexpr size_t kPacketMax = W4_ALLREDUCE_LL_MAX_BYTES;

enum
{
    kOneShotPackets = 0,
    kTwoShotPackets = 1,
    kTwoShotFlags = 2
};

// One copy of the data areas: [packets A: world slots][packets B: world slots][plain inbox: world
// slots][reduced]. The last two are empty when no message can exceed W4_ALLREDUCE_LL_MAX_BYTES.
struct Layout
{
    size_t pkt_slot;     // one sender's slot in either packet inbox
    size_t plain_slot;   // one sender's slot in the plain inbox
    size_t reduced;      // reduced-slice buffer
    size_t copy_bytes;   // all areas of one copy
    size_t total;
};

__host__ __device__ inline size_t align256(size_t v)
{
    return (v + 255) & ~size_t(255);
}

__host__ __device__ inline Layout layout_for(size_t max_bytes, int world)
{
    Layout l;
    size_t const one = max_bytes < kOneShotMax ? max_bytes : kOneShotMax;     // whole message per sender
    size_t const pk = max_bytes < kPacketMax ? max_bytes : kPacketMax;
    size_t const pk_slice = (pk + world - 1) / world + 16;                    // one slice per sender
    l.pkt_slot = align256(2 * (one > pk_slice ? one : pk_slice));            // packets double the bytes
    bool const plain = max_bytes > kPacketMax;
    size_t const slice = (max_bytes + world - 1) / world + 16;
    l.plain_slot = plain ? align256(slice) : 0;
    l.reduced = plain ? align256(slice) : 0;
    l.copy_bytes = 2 * world * l.pkt_slot + world * l.plain_slot + l.reduced;
    l.total = kHeaderBytes + 2 * l.copy_bytes;
    return l;
}

struct RankArgs
{
    void const* partial;
    uint8_t* ws[kMaxRanks]; // ws[r]: rank r's workspace block as mapped into this process
    void const* bias;
    void* out;
    size_t count;
    int n;
    int rank;
};

struct Batch
{
    RankArgs r[kMaxRanks]; // one entry per rank served by this launch (1 in production)
    int ranks_in_launch;
    int ctas_per_rank;
    int world;
    int protocol;
    int skip_push; // one-shot packets only: the GEMM in front has already sent this rank's packets
    size_t pkt_slot, plain_slot, copy_bytes;
    unsigned long long timeout_ns;
};

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(uint32_t const* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Data that another GPU writes (inboxes) or owns (reduced) is accessed around L1.
__device__ __forceinline__ uint4 ld_sys(void const* p)
{
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ void st_sys(void* p, uint4 v)
{
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// One 16-byte vector of data as two flagged packets at dst[0], dst[1].
__device__ __forceinline__ void put_packets(uint4* dst, uint4 v, uint32_t epoch)
{
    st_sys(dst, make_uint4(v.x, epoch, v.y, epoch));
    st_sys(dst + 1, make_uint4(v.z, epoch, v.w, epoch));
}

// Polls the packet pairs at inbox + r * slot + 32 * vec for every rank r in `mask` until all carry
// `epoch`; v[r] receives the data. False when the time limit expired (here or in another thread).
__device__ __forceinline__ bool get_packets(uint4 (&v)[kMaxRanks], uint8_t const* inbox, size_t slot, size_t vec,
    uint32_t mask, uint32_t epoch, unsigned long long timeout_ns, volatile int* failed)
{
    unsigned long long t0 = 0;
    for (uint32_t polls = 1;; ++polls)
    {
        // all loads are issued before the first flag is looked at
        uint32_t bad = 0;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (mask >> r & 1u)
            {
                uint4 const* src = reinterpret_cast<uint4 const*>(inbox + size_t(r) * slot) + 2 * vec;
                uint4 const p0 = ld_sys(src), p1 = ld_sys(src + 1);
                v[r] = make_uint4(p0.x, p0.z, p1.x, p1.z);
                bad |= (p0.y ^ epoch) | (p0.w ^ epoch) | (p1.y ^ epoch) | (p1.w ^ epoch);
            }
        if (bad == 0)
            return true;
        if ((polls & 15u) == 0)
        {
            if (*failed)
                return false;
            unsigned long long const now = global_timer_ns();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > timeout_ns)
            {
                *failed = 1;
                atomicExch(&g_device_status, kDeviceTimeout);
                return false;
            }
        }
    }
}

// dst[i] = src[i] for i in [v0, v1), four 16-byte vectors in flight per thread (NVLink needs about a
// megabyte in flight per GPU to run at full rate). PEER_SRC: the source is another GPU's memory.
template <bool PEER_SRC>
__device__ __forceinline__ void copy_vectors(uint4* dst, uint4 const* src, size_t v0, size_t v1)
{
    size_t i = v0 + threadIdx.x;
    for (; i + 3 * kThreads < v1; i += 4 * kThreads)
    {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            v[u] = PEER_SRC ? ld_sys(src + i + u * kThreads) : src[i + u * kThreads];
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            if (PEER_SRC)
                dst[i + u * kThreads] = v[u];
            else
                st_sys(dst + i + u * kThreads, v[u]);
        }
    }
    for (; i < v1; i += kThreads)
    {
        if (PEER_SRC)
            dst[i] = ld_sys(src + i);
        else
            st_sys(dst + i, src[i]);
    }
}

template <typename T>
__device__ __forceinline__ void add8(float (&acc)[8], uint4 v)
{
    uint32_t const w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        float lo, hi;
        Pair<T>::unpack2(w[j], lo, hi);
        acc[2 * j] += lo;
        acc[2 * j + 1] += hi;
    }
}

template <typename T>
__device__ __forceinline__ uint4 pack8(float const (&acc)[8])
{
    using P = Pair<T>;
    uint4 o;
    o.x = uint32_t(P::from_float(acc[0])) | (uint32_t(P::from_float(acc[1])) << 16);
    o.y = uint32_t(P::from_float(acc[2])) | (uint32_t(P::from_float(acc[3])) << 16);
    o.z = uint32_t(P::from_float(acc[4])) | (uint32_t(P::from_float(acc[5])) << 16);
    o.w = uint32_t(P::from_float(acc[6])) | (uint32_t(P::from_float(acc[7])) << 16);
    return o;
}

// Sum over ranks 0..world-1 in rank order (+ bias vector), rounded to T: v[r] from the peers, `mine`
// in this rank's place.
template <typename T>
__device__ __forceinline__ uint4 sum_ranks(uint4 const (&v)[kMaxRanks], uint4 mine, int rank, int world,
    uint4 const* bias_vec)
{
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
        if (r < world)
            add8<T>(acc, r == rank ? mine : v[r]);
    if (bias_vec)
        add8<T>(acc, __ldg(bias_vec));
    return pack8<T>(acc);
}

// Waits (threads 0..world-1, one flag word each) until every peer's flag for this chunk has reached
// `epoch`; returns false for the whole CTA when the time limit expired.
__device__ __forceinline__ bool wait_peers(uint32_t const* flags, int world, int rank, int chunk, uint32_t epoch,
    unsigned long long timeout_ns, int* failed)
{
    if (int(threadIdx.x) < world && int(threadIdx.x) != rank)
    {
        uint32_t const* word = flags + size_t(threadIdx.x) * kMaxCtas + chunk;
        unsigned long long const t0 = global_timer_ns();
        uint32_t polls = 0;
        while (int32_t(ld_acquire_sys(word) - epoch) < 0)
        {
            if ((++polls & 63u) == 0 && global_timer_ns() - t0 > timeout_ns)
            {
                *failed = 1;
                atomicExch(&g_device_status, kDeviceTimeout);
                break;
            }
        }
    }
    __syncthreads();
    return *failed == 0;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) allreduce_kernel(Batch const b)
{
    __shared__ int failed;
    int const which = int(blockIdx.x) / b.ctas_per_rank; // which of the launch's ranks this CTA serves
    int const c = int(blockIdx.x) - which * b.ctas_per_rank;
    int const C = b.ctas_per_rank;
    RankArgs const& a = b.r[which];
    int const world = b.world, rank = a.rank;
    uint8_t* const mine = a.ws[rank];
    uint32_t* const ctrl = reinterpret_cast<uint32_t*>(mine);

    if (threadIdx.x == 0)
        failed = 0;
    // Programmatic dependent launch: the kernel that follows on the stream may start its prologue now
    // (the decode GEMM fetches its weights meanwhile); this kernel itself may have been started before
    // the one in front has finished, and touches nothing (not even the call number, which the previous
    // all-reduce call two kernels back may still be about to advance) before that one is complete.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Call number: read by every CTA before any CTA of this launch can advance it (see the end).
    uint32_t const epoch = *reinterpret_cast<volatile uint32_t*>(ctrl) + 1u;
    int const h = int(epoch & 1u);
    __syncthreads();

    auto flags_of = [&](uint8_t* ws, int set) // set 0: arrival flags, set 1: "reduced slice published"
    { return reinterpret_cast<uint32_t*>(ws + kCtrlBytes + size_t(set) * kFlagBytes) + size_t(h) * kMaxRanks * kMaxCtas; };
    auto copy_of = [&](uint8_t* ws) { return ws + kHeaderBytes + size_t(h) * b.copy_bytes; };
    auto packets_of = [&](uint8_t* ws, int inbox) { return copy_of(ws) + size_t(inbox) * world * b.pkt_slot; };
    auto plain_of = [&](uint8_t* ws, int sender)
    { return copy_of(ws) + size_t(2) * world * b.pkt_slot + size_t(sender) * b.plain_slot; };
    auto reduced_of = [&](uint8_t* ws) { return copy_of(ws) + size_t(2) * world * b.pkt_slot + size_t(world) * b.plain_slot; };

    size_t const V = a.count / 8; // 16-byte vectors in the message
    int const n_vec = a.n / 8;
    uint4 const* partial = static_cast<uint4 const*>(a.partial);
    uint4 const* bias = static_cast<uint4 const*>(a.bias);
    uint4* out = static_cast<uint4*>(a.out);
    uint32_t const peers = ((1u << world) - 1u) & ~(1u << rank);
    // slice j = vectors [V j / world, V (j+1) / world)
    auto slice_begin = [&](int j) { return V * size_t(j) / world; };

    if (b.protocol == kOneShotPackets)
    {
        size_t const v0 = V * size_t(c) / C, v1 = V * size_t(c + 1) / C;
        for (size_t i = v0 + threadIdx.x; !b.skip_push && i < v1; i += blockDim.x)
        {
            uint4 const v = partial[i];
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p)
                if (peers >> p & 1u)
                    put_packets(reinterpret_cast<uint4*>(packets_of(a.ws[p], 0) + size_t(rank) * b.pkt_slot) + 2 * i, v, epoch);
        }
        for (size_t i = v0 + threadIdx.x; i < v1; i += blockDim.x)
        {
            uint4 v[kMaxRanks];
            if (!get_packets(v, packets_of(mine, 0), b.pkt_slot, i, peers, epoch, b.timeout_ns, &failed))
                break;
            out[i] = sum_ranks<T>(v, partial[i], rank, world, bias ? bias + (i % n_vec) : nullptr);
        }
    }
    else if (b.protocol == kTwoShotPackets)
    {
        // Every slice is cut into the same C chunks of vector indices (slices differ by at most one
        // vector in length; the index range is that of the longest).
        size_t const max_len = (V + world - 1) / world;
        size_t const v0 = max_len * size_t(c) / C, v1 = max_len * size_t(c + 1) / C;
        size_t const s0 = slice_begin(rank), len = slice_begin(rank + 1) - s0;
        // ---- vectors of slice j go to its owner j, inbox A, slot `rank`
        for (size_t i = v0 + threadIdx.x; i < v1; i += blockDim.x)
        {
#pragma unroll
            for (int dj = 1; dj < kMaxRanks; ++dj)
            {
                int const j = (rank + dj) % world; // start with the next rank: spreads the traffic
                if (dj < world)
                {
                    size_t const t0 = slice_begin(j), tl = slice_begin(j + 1) - t0;
                    if (i < tl)
                        put_packets(reinterpret_cast<uint4*>(packets_of(a.ws[j], 0) + size_t(rank) * b.pkt_slot) + 2 * i,
                            partial[t0 + i], epoch);
                }
            }
        }
        // ---- reduce the own slice, write it out and send it to every peer's inbox B, slot `rank`
        bool ok = true;
        for (size_t i = v0 + threadIdx.x; i < v1 && i < len; i += blockDim.x)
        {
            uint4 v[kMaxRanks];
            ok = get_packets(v, packets_of(mine, 0), b.pkt_slot, i, peers, epoch, b.timeout_ns, &failed);
            if (!ok)
                break;
            uint4 const o = sum_ranks<T>(v, partial[s0 + i], rank, world, bias ? bias + ((s0 + i) % n_vec) : nullptr);
            out[s0 + i] = o;
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p)
                if (peers >> p & 1u)
                    put_packets(reinterpret_cast<uint4*>(packets_of(a.ws[p], 1) + size_t(rank) * b.pkt_slot) + 2 * i, o, epoch);
        }
        // ---- collect the other slices from inbox B
        for (size_t i = v0 + threadIdx.x; ok && i < v1; i += blockDim.x)
        {
            uint32_t mask = 0;
#pragma unroll
            for (int j = 0; j < kMaxRanks; ++j)
                if ((peers >> j & 1u) && i < slice_begin(j + 1) - slice_begin(j))
                    mask |= 1u << j;
            uint4 v[kMaxRanks];
            if (!get_packets(v, packets_of(mine, 1), b.pkt_slot, i, mask, epoch, b.timeout_ns, &failed))
                break;
#pragma unroll
            for (int j = 0; j < kMaxRanks; ++j)
                if (mask >> j & 1u)
                    out[slice_begin(j) + i] = v[j];
        }
    }
    else
    {
        bool ok = true;
        // ---- phase 1: push chunk c of slice j to its owner j, slot `rank`, at the slice-relative offset
        for (int dj = 1; dj < world; ++dj)
        {
            int const j = (rank + dj) % world;
            size_t const s0 = slice_begin(j), len = slice_begin(j + 1) - s0;
            size_t const v0 = len * size_t(c) / C, v1 = len * size_t(c + 1) / C;
            copy_vectors<false>(reinterpret_cast<uint4*>(plain_of(a.ws[j], rank)), partial + s0, v0, v1);
        }
        __syncthreads();
        if (int(threadIdx.x) < world && int(threadIdx.x) != rank)
        {
            __threadfence_system();
            st_release_sys(flags_of(a.ws[threadIdx.x], 0) + size_t(rank) * kMaxCtas + c, epoch);
        }
        // ---- phase 2: reduce chunk c of the own slice, publish it
        size_t const s0 = slice_begin(rank), len = slice_begin(rank + 1) - s0;
        size_t const v0 = len * size_t(c) / C, v1 = len * size_t(c + 1) / C;
        ok = wait_peers(flags_of(mine, 0), world, rank, c, epoch, b.timeout_ns, &failed);
        if (ok)
        {
            uint4* red = reinterpret_cast<uint4*>(reduced_of(mine));
            for (size_t i = v0 + threadIdx.x; i < v1; i += kThreads)
            {
                uint4 v[kMaxRanks];
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r)
                    if (peers >> r & 1u)
                        v[r] = ld_sys(reinterpret_cast<uint4 const*>(plain_of(mine, r)) + i);
                uint4 const o = sum_ranks<T>(v, partial[s0 + i], rank, world, bias ? bias + ((s0 + i) % n_vec) : nullptr);
                st_sys(red + i, o);
                out[s0 + i] = o;
            }
        }
        __syncthreads();
        if (ok && int(threadIdx.x) < world && int(threadIdx.x) != rank)
        {
            __threadfence_system();
            st_release_sys(flags_of(a.ws[threadIdx.x], 1) + size_t(rank) * kMaxCtas + c, epoch);
        }
        // ---- phase 3: pull chunk c of every other slice from its owner
        if (ok)
            ok = wait_peers(flags_of(mine, 1), world, rank, c, epoch, b.timeout_ns, &failed);
        if (ok)
        {
            for (int dj = 1; dj < world; ++dj)
            {
                int const j = (rank + dj) % world;
                size_t const t0 = slice_begin(j), tl = slice_begin(j + 1) - t0;
                size_t const w0 = tl * size_t(c) / C, w1 = tl * size_t(c + 1) / C;
                copy_vectors<true>(out + t0, reinterpret_cast<uint4 const*>(reduced_of(a.ws[j])), w0, w1);
            }
        }
    }

    // ---- the last CTA of this rank's launch advances the call number
    __syncthreads();
    // (No fences: every CTA has read the number before it takes its ticket, and the next call is a
    // later kernel on the stream, which sees everything this one wrote.)
    if (threadIdx.x == 0)
    {
        uint32_t const ticket = atomicAdd(ctrl + 1, 1u);
        if (ticket == uint32_t(C) - 1u)
        {
            ctrl[1] = 0u;
            *reinterpret_cast<volatile uint32_t*>(ctrl) = epoch;
        }
    }
}

static int check_one(W4AllReduceParams const& p)
{
    if (!p.out || !p.partial)
        return W4_ERR_NULL_POINTER;
    if (p.world < 1 || p.world > kMaxRanks || p.rank < 0 || p.rank >= p.world)
        return W4_ERR_BAD_SHAPE;
    if (p.act_dtype != W4_DTYPE_FP16 && p.act_dtype != W4_DTYPE_BF16)
        return W4_ERR_BAD_DTYPE;
    if (p.mode != W4_ALLREDUCE_AUTO && p.mode != W4_ALLREDUCE_ONE_SHOT && p.mode != W4_ALLREDUCE_TWO_SHOT
        && p.mode != W4_ALLREDUCE_GATHER_ONLY)
        return W4_ERR_BAD_REGIME;
    if (p.count % 8 != 0 || p.n <= 0 || p.n % 8 != 0 || p.count % size_t(p.n) != 0)
        return W4_ERR_BAD_SHAPE;
    for (int r = 0; r < p.world; ++r)
    {
        if (!p.workspace[r])
            return W4_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(p.workspace[r]) & 255u)
            return W4_ERR_MISALIGNED;
    }
    if ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.bias) | reinterpret_cast<uintptr_t>(p.partial))
        & 15u)
        return W4_ERR_MISALIGNED;
    return W4_OK;
}

// 1 = two-shot. AUTO follows the reference's size rule for its one-shot kernel
// (allreducePlugin.cpp:258-283): always up to 2 ranks, below 1 MB up to 4, below 500 kB beyond.
static int pick_two_shot(int mode, size_t bytes, int world)
{
    if (world == 1 || mode == W4_ALLREDUCE_ONE_SHOT || mode == W4_ALLREDUCE_GATHER_ONLY)
        return 0;
    if (mode == W4_ALLREDUCE_TWO_SHOT)
        return 1;
    if (bytes > size_t(W4_ONESHOT_MAX_BYTES))
        return 1;
    if (world <= 2)
        return 0;
    return bytes < (world <= 4 ? size_t(1000000) : size_t(500000)) ? 0 : 1;
}

static bool layout_from_workspace(W4AllReduceParams const& p, size_t bytes, Layout* l)
{
    // The workspace was sized for some largest message: recover the layout from its size (capacity is
    // monotone in the largest message, so search for the largest one whose layout fits).
    size_t lo = 0, hi = size_t(1) << 34;
    while (lo < hi)
    {
        size_t const mid = lo + (hi - lo + 1) / 2;
        if (layout_for(mid, p.world).total <= p.workspace_bytes)
            lo = mid;
        else
            hi = mid - 1;
    }
    if (lo < bytes || p.workspace_bytes <= kHeaderBytes)
        return false;
    *l = layout_for(lo, p.world);
    return true;
}

static int launch(W4AllReduceParams const* ranks, int ranks_in_launch, cudaStream_t stream)
{
    W4AllReduceParams const& p0 = ranks[0];
    size_t const bytes = p0.count * 2;
    Batch b{};
    b.world = p0.world;
    b.ranks_in_launch = ranks_in_launch;
    bool const two_shot = pick_two_shot(p0.mode, bytes, p0.world) != 0;
    if (!two_shot && bytes > kOneShotMax)
        return W4_ERR_UNSUPPORTED; // a one-shot message must fit one sender slot
    b.protocol = bytes > kPacketMax ? kTwoShotFlags : (two_shot ? kTwoShotPackets : kOneShotPackets);
    b.skip_push = p0.mode == W4_ALLREDUCE_GATHER_ONLY ? 1 : 0;
    // The caller passes what w4_allreduce_workspace_bytes(max_bytes, world) returned.
    Layout l{};
    if (!layout_from_workspace(p0, bytes, &l))
        return W4_ERR_WORKSPACE;
    b.pkt_slot = l.pkt_slot;
    b.plain_slot = l.plain_slot;
    b.copy_bytes = l.copy_bytes;
    b.timeout_ns = p0.timeout_ms > 0 ? (unsigned long long) (p0.timeout_ms) * 1000000ull : 2000000000ull;

    w4::DeviceInfo const& dev = w4::current_device_info();
    if (dev.num_sms <= 0)
        return W4_ERR_CUDA;
    // Chunks: at most kMaxCtas; all ranks derive the same number from the message size alone. The
    // packet protocols are bound by how fast one SM issues stores towards the peers (2 * (world - 1)
    // per vector: measured about 30 cycles per warp-wide store), so their work is spread thin: 128
    // vectors per CTA of 128 threads. The flag protocol moves whole chunks: 512 threads, 8 KB or more
    // each. Several ranks in one launch (single-GPU emulation) must all be resident at once, so the
    // number is capped by the SMs available per rank.
    size_t const vecs = p0.count / 8;
    size_t const unit = b.protocol == kOneShotPackets ? vecs : (vecs + p0.world - 1) / p0.world;
    int const cap = kMaxCtas < dev.num_sms / ranks_in_launch ? kMaxCtas : dev.num_sms / ranks_in_launch;
    if (cap < 1)
        return W4_ERR_UNSUPPORTED;
    int threads = kThreads;
    int ctas = int(unit / kThreads);
    if (b.protocol != kTwoShotFlags)
    {
        threads = kPacketThreads;
        ctas = int((unit + kPacketThreads - 1) / kPacketThreads);
        if (ctas > cap) // more work than thin CTAs can cover: full-size CTAs
        {
            threads = kThreads;
            ctas = int((unit + kThreads - 1) / kThreads);
        }
    }
    ctas = ctas < 1 ? 1 : (ctas > cap ? cap : ctas);
    b.ctas_per_rank = ctas;
    for (int i = 0; i < ranks_in_launch; ++i)
    {
        W4AllReduceParams const& p = ranks[i];
        RankArgs& a = b.r[i];
        a.partial = p.partial;
        for (int r = 0; r < p.world; ++r)
            a.ws[r] = static_cast<uint8_t*>(p.workspace[r]);
        a.bias = p.bias;
        a.out = p.out;
        a.count = p.count;
        a.n = p.n;
        a.rank = p.rank;
    }
    dim3 const grid(unsigned(ctas * ranks_in_launch)), block(threads);
    void* args[] = {&b};
    cudaError_t rc;
    if (ranks_in_launch > 1)
    {
        // CTAs of different emulated ranks wait for one another: they must be co-resident.
        rc = p0.act_dtype == W4_DTYPE_FP16
            ? cudaLaunchCooperativeKernel(reinterpret_cast<void*>(allreduce_kernel<__half>), grid, block, args, 0, stream)
            : cudaLaunchCooperativeKernel(reinterpret_cast<void*>(allreduce_kernel<__nv_bfloat16>), grid, block, args, 0,
                stream);
    }
    else
    {
        // A programmatic dependent of whatever precedes it in the stream (see the kernel's first lines).
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        rc = p0.act_dtype == W4_DTYPE_FP16 ? cudaLaunchKernelEx(&cfg, allreduce_kernel<__half>, b)
                                           : cudaLaunchKernelEx(&cfg, allreduce_kernel<__nv_bfloat16>, b);
        if (rc == cudaSuccess)
            rc = cudaGetLastError();
    }
    return rc == cudaSuccess ? W4_OK : W4_ERR_CUDA;
}

} // namespace ar

bool allreduce_push_target(W4AllReduceParams const& r, PushTarget* t)
{
    if (ar::check_one(r) != W4_OK)
        return false;
    size_t const bytes = r.count * 2;
    if (r.mode == W4_ALLREDUCE_TWO_SHOT || bytes > ar::kOneShotMax || ar::pick_two_shot(r.mode, bytes, r.world) != 0)
        return false; // only the one-shot packet protocol takes packets from the GEMM
    ar::Layout l{};
    if (!ar::layout_from_workspace(r, bytes, &l))
        return false;
    for (int i = 0; i < W4_MAX_RANKS; ++i)
        t->ws[i] = i < r.world ? static_cast<uint8_t*>(r.workspace[i]) : nullptr;
    t->rank = r.rank;
    t->world = r.world;
    t->pkt_slot = l.pkt_slot;
    t->copy_bytes = l.copy_bytes;
    t->header_bytes = ar::kHeaderBytes;
    t->gather = 0;
    t->bias = nullptr;
    t->timeout_ns = r.timeout_ms > 0 ? (unsigned long long) (r.timeout_ms) * 1000000ull : 2000000000ull;
    return true;
}

} // namespace w4

extern "C" size_t w4_allreduce_workspace_bytes(size_t max_message_bytes, int world)
{
    if (world < 1 || world > w4::ar::kMaxRanks || max_message_bytes == 0)
        return 0;
    return w4::ar::layout_for(max_message_bytes, world).total;
}

extern "C" int w4_allreduce(const W4AllReduceParams* p, void* stream)
{
    if (!p)
        return W4_ERR_NULL_POINTER;
    int const rc = w4::ar::check_one(*p);
    if (rc != W4_OK)
        return rc;
    if (p->count == 0)
        return W4_OK;
    return w4::ar::launch(p, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int w4_allreduce_emulated(const W4AllReduceParams* ranks, int world, void* stream)
{
    if (!ranks)
        return W4_ERR_NULL_POINTER;
    if (world < 1 || world > w4::ar::kMaxRanks)
        return W4_ERR_BAD_SHAPE;
    for (int r = 0; r < world; ++r)
    {
        int const rc = w4::ar::check_one(ranks[r]);
        if (rc != W4_OK)
            return rc;
        if (ranks[r].world != world || ranks[r].rank != r || ranks[r].count != ranks[0].count
            || ranks[r].act_dtype != ranks[0].act_dtype || ranks[r].mode != ranks[0].mode
            || ranks[r].workspace_bytes != ranks[0].workspace_bytes)
            return W4_ERR_BAD_SHAPE;
    }
    if (ranks[0].count == 0)
        return W4_OK;
    return w4::ar::launch(ranks, world, static_cast<cudaStream_t>(stream));
}
