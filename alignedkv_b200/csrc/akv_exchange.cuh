// Device side of the exchange of the shards' packed results through peer memory, fused with their log-sum-exp merge
// (sequence-sharded decode, one process per GPU of one node; no counterpart in the reference, which is single-device).
//
// Every rank owns one exchange buffer in its own device memory and maps the buffers of the other ranks (CUDA IPC
// over NVLink).  Layout of a buffer for R ranks, `rows` (batch, query head) rows and W = head_dim + 2 floats per record:
//     float    data [2][R][rows][W]      records (m, l, o[0..D-1]) as written by rank g into slot g, two epochs deep
//     uint32_t flags[2][R][rows]         at byte offset exchange_data_bytes(): the epoch whose record is complete
// Once per decode step on every rank, one CTA per row (exchange_merge_row):
//   1. publish - the CTA stores its row's record into slot `rank` of EVERY rank's buffer (plain stores, this GPU's
//      memory and the peers'), then one thread per peer orders them (__threadfence_system) and stores the epoch into
//      that peer's flag with release semantics at system scope;
//   2. wait - one thread per source rank polls ITS OWN buffer's flag (acquire, system scope) until it holds the epoch.
//      The wait is time-bounded: when it runs out the CTA raises the library's device error flag, writes zeros
//      and returns, so the context stays usable;
//   3. merge - the row's R records are combined (lse_merge_row) and written as fp16.
// Two epochs deep is enough: a rank can only leave step k after every peer has published step k, which a peer does
// after its own step k-1 has completed; so a record of step k+1 never lands on one of step k-1 that is still read.
// The polling reads memory of this GPU only; nothing here uses multicast, and peers are touched by plain stores only.
#pragma once
#include "akv_common.cuh"

namespace akv {

constexpr int XCHG_MAX_RANKS = 8;

struct XchgParams {
    uint8_t* bufs[XCHG_MAX_RANKS];   // this process's addresses of every rank's buffer (its own at [rank])
    __half* out;                     // merged output [rows][D]
    unsigned int* err;               // the device error flag of the exchange (bit 2 is raised when a wait ran out)
    unsigned long long timeout_ns;
    int rank, R, rows, D;            // R == 0: no exchange
    uint32_t epoch;                  // the same on every rank, one more per step, never 0
};

__host__ __device__ inline size_t exchange_data_bytes(int R, int rows, int D) {
    return ((size_t)2 * R * rows * (D + 2) * sizeof(float) + 127) & ~(size_t)127;
}

__device__ __forceinline__ unsigned long long xchg_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Row i of the step: publishes src[0..D+2) (global memory, complete and visible to the whole CTA: the caller has
// passed a CTA barrier since it was written), waits for the other ranks' records and writes the merged row.
// Called by every thread of the CTA (at least XCHG_MAX_RANKS threads); s_buf: XCHG_MAX_RANKS pointers of shared memory.
__device__ __forceinline__ void exchange_merge_row(const XchgParams& p, const float* src, int i, uint8_t** s_buf) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int W = p.D + 2, R = p.R;
    const uint32_t par = p.epoch & 1u;
    const size_t fl0 = exchange_data_bytes(R, p.rows, p.D);
    if (tid < XCHG_MAX_RANKS) {
        uint8_t* mine = nullptr;                   // (selected, not indexed: the parameter array stays out of local memory)
#pragma unroll
        for (int g = 0; g < XCHG_MAX_RANKS; ++g) mine = tid == g ? p.bufs[g] : mine;
        s_buf[tid] = mine;
    }
    __syncthreads();
    const size_t slot = (((size_t)par * R + p.rank) * p.rows + i) * W;          // in floats
    for (int idx = tid; idx < R * W; idx += nt) {
        const int g = idx / W, c = idx - g * W;
        reinterpret_cast<float*>(s_buf[g])[slot + c] = src[c];
    }
    __syncthreads();
    bool ok = true;
    if (tid < R) {
        __threadfence_system();
        uint32_t* theirs = reinterpret_cast<uint32_t*>(s_buf[tid] + fl0) + ((size_t)par * R + p.rank) * p.rows + i;
        st_release_sys(theirs, p.epoch);
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(s_buf[p.rank] + fl0) + ((size_t)par * R + tid) * p.rows + i;
        const unsigned long long t0 = xchg_now_ns();
        while (ld_acquire_sys(mine) != p.epoch) {
            if (xchg_now_ns() - t0 > p.timeout_ns) { ok = false; break; }
            __nanosleep(64);
        }
    }
    ok = __syncthreads_and(ok);
    __half* out = p.out + (size_t)i * p.D;
    if (!ok) {
        if (tid == 0) atomicOr(p.err, 4u);
        for (int d = tid; d < p.D; d += nt) out[d] = __float2half_rn(0.f);
        return;
    }
    const float* base = reinterpret_cast<const float*>(s_buf[p.rank]) + ((size_t)par * R * p.rows + i) * W;
    lse_merge_row(base, (size_t)p.rows * W, R, p.D, out, tid, nt);
}

// Host side (akv_exchange.cu): checks the arguments of an exchange and fills the kernel parameters.
int fill_exchange(XchgParams* p, void* const* bufs, int rank, int n_ranks, void* out, int rows, int head_dim,
                  unsigned int epoch, int timeout_ms);

}  // namespace akv
