// Device side of the exchange of the shards' packed results through peer memory, fused with their log-sum-exp merge
// (sequence-sharded decode, one process per GPU of one node; no counterpart in the reference, which is single-device).
//
// Every rank owns one exchange buffer in its own device memory and maps the buffers of the other ranks (CUDA IPC
// over NVLink).  A buffer for R ranks, `rows` (batch, query head) rows and W = head_dim + 2 floats per record is
//     uint2 words[2][R][rows][W]     word = (bits of one float of the record (m, l, o[0..D-1]), epoch it belongs to);
//                                    slot g is written by rank g; two epochs deep (index = epoch & 1)
// Every float travels with its own flag in ONE aligned 8-byte store, which is atomic: a reader that finds the epoch
// in a word has the value too, so neither side needs a fence (a system-scope fence costs microseconds, and this
// exchange sits on the critical path of every decode step).  Once per step on every rank, one CTA per row
// (exchange_merge_row):
//   1. publish - the CTA stores its row's record, word by word, into slot `rank` of EVERY rank's buffer (volatile
//      8-byte stores: this GPU's memory and the peers');
//   2. collect - the CTA's threads read the R x W words of the row from THEIR OWN buffer (volatile 8-byte loads, local
//      memory only), each word until it carries the step's epoch, into shared memory.  The wait is time-bounded: when
//      it runs out the CTA raises the library's device error flag, writes zeros and returns, so the context stays
//      usable;
//   3. merge - the row's R records are combined (lse_merge_row) and written as fp16.
// Two epochs deep is enough: a rank can only leave step k after every peer has published step k, which a peer does
// after its own step k-1 has completed; so a word of step k+1 never lands on one of step k-1 that is still awaited.
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

constexpr int XCHG_MAX_D = 256;                      // head_dim limit of the exchange (the collected row lives in shared memory)
constexpr int XCHG_ROW_FLOATS = XCHG_MAX_RANKS * (XCHG_MAX_D + 2);

__host__ __device__ inline size_t exchange_buffer_bytes(int R, int rows, int D) {
    return (size_t)2 * R * rows * (D + 2) * sizeof(uint2);
}

__device__ __forceinline__ unsigned long long xchg_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_word(uint2* p, uint32_t v, uint32_t e) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};\n" ::"l"(p), "r"(v), "r"(e) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// Row i of the step: publishes src[0..D+2) (global memory, complete and visible to the whole CTA: the caller has
// passed a CTA barrier since it was written), collects the R records of the row and writes the merged row.
// Called by every thread of the CTA (at least XCHG_MAX_RANKS threads).  Shared memory: s_buf, XCHG_MAX_RANKS pointers;
// s_rec, XCHG_ROW_FLOATS floats.
__device__ __forceinline__ void exchange_merge_row(const XchgParams& p, const float* src, int i, uint8_t** s_buf,
                                                   float* s_rec) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int W = p.D + 2, R = p.R;
    const uint32_t par = p.epoch & 1u;
    if (tid < XCHG_MAX_RANKS) {
        uint8_t* mine = nullptr;                   // (selected, not indexed: the parameter array stays out of local memory)
#pragma unroll
        for (int g = 0; g < XCHG_MAX_RANKS; ++g) mine = tid == g ? p.bufs[g] : mine;
        s_buf[tid] = mine;
    }
    __syncthreads();
    const size_t slot = (((size_t)par * R + p.rank) * p.rows + i) * W;          // in words
    for (int idx = tid; idx < R * W; idx += nt) {
        const int g = idx / W, c = idx - g * W;
        st_word(reinterpret_cast<uint2*>(s_buf[g]) + slot + c, __float_as_uint(src[c]), p.epoch);
    }
    const uint2* own = reinterpret_cast<const uint2*>(s_buf[p.rank]);
    bool ok = true;
    const int n = R * W;
    for (int base = tid; base < n; base += 4 * nt) {
        // four words in flight per thread; one that does not carry the epoch yet is then awaited by itself
        const uint2* w[4];
        uint2 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = base + u * nt;
            const int g = idx / W, c = idx - g * W;
            w[u] = own + (((size_t)par * R + g) * p.rows + i) * W + c;
            if (idx < n) v[u] = ld_word(w[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = base + u * nt;
            if (idx >= n || !ok) continue;
            if (v[u].y != p.epoch) {
                const unsigned long long t0 = xchg_now_ns();
                for (;;) {
                    __nanosleep(20);
                    v[u] = ld_word(w[u]);
                    if (v[u].y == p.epoch) break;
                    if (xchg_now_ns() - t0 > p.timeout_ns) { ok = false; break; }
                }
            }
            s_rec[idx] = __uint_as_float(v[u].x);
        }
    }
    ok = __syncthreads_and(ok);
    __half* out = p.out + (size_t)i * p.D;
    if (!ok) {
        if (tid == 0) atomicOr(p.err, 4u);
        for (int d = tid; d < p.D; d += nt) out[d] = __float2half_rn(0.f);
        return;
    }
    lse_merge_row([&](int g, int c) { return s_rec[g * W + c]; }, R, p.D, out, tid, nt);
}

// Host side (akv_exchange.cu): checks the arguments of an exchange and fills the kernel parameters.
int fill_exchange(XchgParams* p, void* const* bufs, int rank, int n_ranks, void* out, int rows, int head_dim,
                  unsigned int epoch, int timeout_ms);

}  // namespace akv
