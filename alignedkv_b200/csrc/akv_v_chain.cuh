// Exact-order P.V, streaming form: the kernel body behind v_cache_compute for head_dim 128.
//
// Replaces the reference's v_cache_compute_kernel (extension/csrc/V_cache.cu:178-308); bit-identical outputs: every
// output channel is the fp16 fused-multiply-add chain over tokens 0..n-1 in order (V_cache.cu:203,304), skipped nibble
// planes are replaced by the reference's constants (V_cache.cu:198-202,250-253).
//
// Design (B200).  The token order leaves one dependent chain per (batch, query head, channel pair); a dependent
// fp16x2 FMA issues every ~4 cycles, so a chain can absorb about 60 GB/s of high bytes per (batch, head) - more than
// a CTA's share of HBM - PROVIDED the chain warp spends its issue slots on little else.  The V layout is token-major
// (a token's 128 high bytes are one row), while a chain thread wants "my channel pair, next tokens".  That
// transposition is done by the load instruction itself: ldmatrix.x4.trans over eight token rows hands every lane the
// 16-bit high-byte pair of ITS channel pair for eight consecutive tokens in four registers.  So the high bytes go
// HBM -> shared memory (one 8 KB bulk asynchronous copy per 64-token stage, exactly as they lie in the plane) ->
// registers of the chain (one ldmatrix + one 16-byte load of probabilities per 8 tokens), and per token the chain
// issues one byte permute (high bytes + the constant low byte 0x80) and one FMA per query head.
//   CTA = one (batch, KV head).  Warps: 2 * G / HPW chain warps + 1 producer warp.
//   chain warp (head group hg, half wh): lane T owns channel pair 32*wh + 8*(T%4) + T/4 (channels 2p, 2p+1) of the
//     HPW query heads hg*HPW .. +HPW-1: HPW independent accumulators that share the high-byte registers.
//   producer warp: per stage it (1) waits until the stage's ring slot was released, (2) starts the 8 KB copy,
//     (3) lane = tokens (lane, lane + 32): takes the probabilities from a buffer bulk-copied a chunk ahead, decides
//     the read codes (V_cache.cu:211,250-251), (4) reserves rows of a small side ring for the tokens whose nibble
//     rows some head of the group reads, records {first side row, union mask, per-head masks} for the chain,
//     (5) starts 64-byte copies of just those nibble rows (one 4 KB copy when the whole stage reads the plane).
//     All copies of a stage are byte-counted on the stage's mbarrier.
//   Groups of 8 tokens in which a head reads a nibble plane (rare in aligned mode: the probability must be within two
//   binades of the probe threshold) take a per-token path that rebuilds the low byte from the side ring; everything
//   else is the lean path above.
// Every wait is bounded (about a second); a wait that runs out raises the device error flag, the chain stores NaN
// instead of a result, and the producer waits (bounded) for its copies in flight before the CTA leaves.
#pragma once
#include "akv_common.cuh"

namespace akv {

struct VParams {
    const uint8_t* first8;
    const uint8_t* mid4;
    const uint8_t* last4;
    const uint16_t* s;      // probabilities, one row per (batch, query head)
    const uint8_t* amin;    // threshold byte per (batch, query head)
    // test_o != nullptr: the kernel computes the threshold bytes itself from the probe result [B,Hq,D] and the
    // exponent maxima [B,H,D] (v_threshold_warp) and stores them to amin_out
    const uint16_t* test_o;
    const uint8_t* v_exp;
    uint8_t* amin_out;
    int H;                  // KV heads
    uint16_t* o;            // [B, Hq, D]
    int max_seq_len, D, s_last_dim, n, reference;
    int group;              // query heads per KV head (1 = multi-head attention)
    int nf, nside, sch;     // streaming form: ring depth (stages), side-ring rows (power of two), stages per chunk
    int units;              // streaming form: number of (batch, KV head) units
    unsigned long long* prof;   // DEBUG
    int dbg;                    // DEBUG
};
static unsigned long long* g_v_prof_host = nullptr;   // DEBUG

// ---- device error flag and shared-memory barriers (mbarrier) with bounded waits
static __device__ unsigned int g_v_wait_gave_up = 0;   // set when a bounded wait ran out (never expected)

__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(a) : "memory");
}
// adds `bytes` to the byte count the current phase waits for (no arrival)
__device__ __forceinline__ void mbar_expect(uint32_t a, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;\n" ::"r"(a), "r"(bytes) : "memory");
}
// arrives and adds `bytes` to the byte count the current phase still waits for
__device__ __forceinline__ void mbar_arrive_expect(uint32_t a, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(a), "r"(bytes) : "memory");
}
// Bounded wait, split so that the common case (the phase has completed, or completes within the hardware's own short
// wait) is a single instruction in the caller's instruction stream and the spin loop lives out of line: the loops that
// call this are latency-critical and must stay compact in the instruction cache.
__device__ __noinline__ bool mbar_wait_slow(uint32_t a, uint32_t parity) {
    unsigned long long t0 = 0;
    for (int spin = 0; spin < (1 << 26); ++spin) {
        uint32_t ok;
        // the hint lets the hardware park the warp (no issue slots taken from the warps that share its scheduler)
        // until the phase completes or the time (ns) runs out
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(a), "r"(parity), "r"(20000u) : "memory");
        if (ok) return true;
        if ((spin & 63) == 63) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > 1000000000ull) break;      // about a second: give up and raise the device error flag
        }
    }
    atomicOr(&g_v_wait_gave_up, 1u);
    return false;
}
// Bounded wait that polls with test_wait (never blocks in hardware) and sleeps between polls.
__device__ __noinline__ bool mbar_wait_sleep(uint32_t a, uint32_t parity, uint32_t ns) {
    unsigned long long t0 = 0;
    for (int spin = 0; spin < (1 << 26); ++spin) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
        __nanosleep(ns);
        if ((spin & 63) == 63) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > 1000000000ull) break;
        }
    }
    atomicOr(&g_v_wait_gave_up, 1u);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t a, uint32_t parity, int* slow = nullptr) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    if (__builtin_expect(ok != 0, 1)) return true;
    if (slow) ++*slow;
    return mbar_wait_slow(a, parity);
}
// Bulk asynchronous copy global -> shared through the TMA unit; 16-byte aligned addresses, size a multiple of 16.
// Completion is signalled on the mbarrier as `bytes` of its pending byte count.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

namespace vch {
constexpr int TOK = 64;            // tokens per stage
constexpr int D = 128, HD = 64;    // head size, bytes of a nibble row
constexpr int F_BYTES = TOK * D;   // high bytes of a stage
__host__ __device__ constexpr int rec_bytes(int G) { return (16 + 8 * G + 15) & ~15; }

// Shared-memory plan (byte offsets), computed the same way on both sides.
struct Plan {
    int f, mid, low, sb, rec, thr, bar, bytes;
};
__host__ __device__ inline Plan plan(int G, int nf, int nside, int sch) {
    Plan p;
    p.f = 0;
    p.mid = nf * F_BYTES;
    p.low = p.mid + nside * HD;
    p.sb = p.low + nside * HD;                 // three probability buffers of G x sch x 64 values
    p.rec = p.sb + 3 * G * sch * TOK * 2;      // per ring slot: {first side row, union mask lo, hi, rows} + per head mask lo, hi
    p.thr = p.rec + nf * rec_bytes(G);         // threshold (already shifted) per head
    p.bar = (p.thr + 4 * G + 7) & ~7;          // full[nf], free[nf], probability buffers[3]
    p.bytes = p.bar + (2 * nf + 3) * 8;
    return p;
}
}  // namespace vch

// Both halves of the result = half `hi ? 1 : 0` of w (the probability of one token for both channels of the pair).
__device__ __forceinline__ __half2 v_dup(uint32_t w, int hi) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    return hi ? __high2half2(h) : __low2half2(h);
}
__device__ __forceinline__ uint32_t v_fma(uint32_t k, __half2 s, uint32_t acc) {
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&k), s, *reinterpret_cast<const __half2*>(&acc));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// Registers of one group of 8 tokens: high-byte pairs [token 2i | token 2i+1] and per head the 8 probabilities.
template <int HPW>
struct VGroup {
    uint32_t h[4];
    uint4 s[HPW];
};
// UPC (batch, KV head) units share a CTA, each with its own warps, rings and barriers.  With two units of four warps
// (G = HPW) the CTA's warps are [chain, chain, copy, decision] x 2 and land one chain warp on each of the SM's four
// schedulers; two independent CTAs of four warps would put both their chain warps on the same two schedulers.
template <int G, int HPW, int UPC, int GPI>
__global__ void __launch_bounds__(UPC * 32 * (2 * G / HPW + 2)) v_chain_kernel(const VParams p) {
    using namespace vch;
    constexpr int NCW = 2 * G / HPW;               // chain warps of a unit; then its copy warp and its decision warp
    constexpr int WPU = NCW + 2;                   // warps per unit
    constexpr int REC = rec_bytes(G);
    static_assert(G % HPW == 0, "heads per warp must divide the group");
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31;
    // warp order inside the CTA: with two units the chain warps come first so that they spread over the schedulers
    const int wcta = tid >> 5;
    const int unit = UPC == 1 ? 0 : (wcta < UPC * NCW ? wcta / NCW : (wcta - UPC * NCW) / 2);
    const int warp = UPC == 1 ? wcta : (wcta < UPC * NCW ? wcta % NCW : NCW + (wcta - UPC * NCW) % 2);
    const long long bh = (long long)blockIdx.x * UPC + unit;   // (batch, KV head)
    const int n = p.n, nf = p.nf, nside = p.nside, sch = p.sch;
    const int nst = (n + TOK - 1) / TOK;
    const Plan pl = plan(G, nf, nside, sch);
    const uint32_t base = smem_u32(smem) + (uint32_t)unit * (uint32_t)((pl.bytes + 127) & ~127);
    const bool unit_on = bh < p.units;
    const uint32_t bar_full = base + pl.bar, bar_free = bar_full + nf * 8, bar_sb = bar_free + nf * 8;
    const uint32_t sb_head = (uint32_t)sch * TOK * 2, sb_buf = sb_head * G;   // bytes of one head's chunk / one buffer

    pdl_enter();
    if (warp == 0 && lane == 0) {
        for (int s = 0; s < nf; ++s) {
            mbar_init(bar_full + s * 8, 2);        // the copy warp's and the decision warp's arrivals (+ the stage's bytes)
            mbar_init(bar_free + s * 8, NCW);      // one arrival per chain warp
        }
        for (int s = 0; s < 3; ++s) mbar_init(bar_sb + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    if (!unit_on) return;                          // (odd number of units: the last CTA's second half has none)

    if (warp == NCW) {
        // ------------------------------------------------------------------ copy warp: the high bytes
        // Stage i -> ring slot i % nf as soon as the chain has released the slot's previous stage: one 8 KB copy,
        // announced on the stage's barrier together with this warp's arrival.
        const uint8_t* F = p.first8 + (size_t)bh * p.max_seq_len * D;
        int slot = 0;
        uint32_t parity = 0;                       // of the release being waited for: (i / nf - 1) & 1
        // The decision warp's first loads (probe result, exponent maxima) go out before this warp floods the memory
        // system with the first ring of copies - behind that flood they would take several times as long, and the
        // first stage cannot be consumed before the thresholds are known.
        asm volatile("bar.sync %0, 64;\n" ::"r"(1 + unit) : "memory");
        bool alive = true;
        int nslow = 0;
        const long long c_t0 = clock64();
        for (int i = 0; i < nst; ++i) {
            if (i >= nf) {
                alive = (p.dbg & 2) ? mbar_wait_sleep(bar_free + slot * 8, parity, 100) : mbar_wait(bar_free + slot * 8, parity, &nslow);
                if (!alive) break;
            }
            if (lane == 0) {
                const int cnt = (n - i * TOK) < TOK ? (n - i * TOK) : TOK;
                const uint32_t bar = bar_full + slot * 8;
                mbar_arrive_expect(bar, (uint32_t)cnt * D);
                bulk_copy(base + pl.f + (uint32_t)slot * F_BYTES, F + (size_t)i * TOK * D, (uint32_t)cnt * D, bar);
            }
            if (++slot == nf) { slot = 0; if (i >= nf) parity ^= 1u; }
        }
        // a wait gave up (never expected): give the copies in flight time to land before the CTA's shared memory is
        // released (a stage completes only with the other warp's arrival, which may not come any more)
        if (!alive) for (int k = 0; k < 1000; ++k) __nanosleep(1000);
        if (p.prof && lane == 0) { p.prof[bh * 16 + 8] = clock64() - c_t0; p.prof[bh * 16 + 9] = nslow; }
        return;
    }
    if (warp == NCW + 1) {
        int nslow_free = 0, nslow_sb = 0;
        const long long d_t0 = clock64();
        long long d_thr = 0;
        // ------------------------------------------------------------------ decision warp: codes, records, nibble rows
        const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * HD;
        const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * HD;
        const uint16_t* s_rows = p.s + (size_t)bh * G * p.s_last_dim;
        bool alive = true;
        // probability chunk c (stages c*sch .. of every head) -> buffer c % 3; issued by one thread
        auto request_s = [&](int c, int buf) {
            const int t0 = c * sch * TOK;
            int cnt = n - t0;
            cnt = cnt > sch * TOK ? sch * TOK : cnt;
            const uint32_t bytes = (uint32_t)((cnt + 7) & ~7) * 2;     // rows are padded to a multiple of 8 values
            const uint32_t bar = bar_sb + buf * 8;
            mbar_arrive_expect(bar, bytes * G);
#pragma unroll
            for (int g = 0; g < G; ++g)
                bulk_copy(base + pl.sb + (uint32_t)buf * sb_buf + g * sb_head, s_rows + (size_t)g * p.s_last_dim + t0,
                          bytes, bar);
        };
        if (lane == 0 && nst > 0) request_s(0, 0);
        // thresholds: from the probe result (decode step) or as given
        uint32_t A[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            uint32_t a;
            if (p.test_o) {
                a = v_threshold_warp(p.test_o, p.v_exp, bh * G + g, p.H, G, D, lane);
                if (lane == 0) p.amin_out[bh * G + g] = (uint8_t)a;
            } else {
                a = p.amin[bh * G + g];
            }
            A[g] = (a << 10) & 0xFFFFu;
            if (lane == 0) asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(base + pl.thr + g * 4), "r"(A[g]) : "memory");
        }
        asm volatile("bar.sync %0, 64;\n" ::"r"(1 + unit) : "memory");
        d_thr = clock64() - d_t0;
        uint32_t side_head = 0, side_tail = 0;    // side rows handed out / taken back so far
        int freed = 0, freed_slot = 0;            // stages whose release has been consumed; freed % nf
        uint32_t freed_parity = 0;                // (freed / nf) & 1
        const uint32_t lt = (1u << lane) - 1u;
        auto reclaim = [&]() {                    // consume the release of stage `freed`: its side rows are free again
            alive = (p.dbg & 2) ? mbar_wait_sleep(bar_free + freed_slot * 8, freed_parity, 100) : mbar_wait(bar_free + freed_slot * 8, freed_parity, &nslow_free);
            side_tail += lds32(base + pl.rec + freed_slot * REC + 12);
            ++freed;
            if (++freed_slot == nf) { freed_slot = 0; freed_parity ^= 1u; }
        };
        int slot = 0, sic = 0, c = 0, cbuf = 0;   // of stage i: i % nf, i % sch, i / sch, (i / sch) % 3
        uint32_t cpar = 0;                        // ((i / sch) / 3) & 1
        for (int i = 0; i < nst && alive; ++i) {
            while (alive && freed <= i - nf) reclaim();
            if (!alive) break;
            if (sic == 0) {             // entering chunk c: ask for the next one, make sure this one has landed
                if ((c + 1) * sch < nst && lane == 0) request_s(c + 1, cbuf == 2 ? 0 : cbuf + 1);
                alive = mbar_wait(bar_sb + cbuf * 8, cpar, &nslow_sb);
                if (!alive) break;
            }
            const int t0 = i * TOK;
            const int cnt = (n - t0) < TOK ? (n - t0) : TOK;
            // read codes of tokens `lane` and `lane + 32` from the bit patterns (V_cache.cu:211,250-251): 16-bit
            // wrap-around, signed compare
            const uint32_t sa = base + pl.sb + (uint32_t)cbuf * sb_buf + (uint32_t)sic * (TOK * 2) + lane * 2;
            uint32_t mm[G][2];
            int uc0 = 2, uc1 = 2;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                // (beyond the last token the buffer holds stale but readable bytes; they are ignored)
                const uint32_t s0 = lds16(sa + g * sb_head), s1 = lds16(sa + g * sb_head + 64);
                const int d0 = (int)(int16_t)(uint16_t)(A[g] - s0), d1 = (int)(int16_t)(uint16_t)(A[g] - s1);
                int c0 = p.reference ? 0 : (d0 >= 0x0800 ? 2 : (d0 >= 0x0400 ? 1 : 0));
                int c1 = p.reference ? 0 : (d1 >= 0x0800 ? 2 : (d1 >= 0x0400 ? 1 : 0));
                if (p.dbg & 4) c0 = c1 = 2;
                if (lane >= cnt) c0 = 2;
                if (lane + 32 >= cnt) c1 = 2;
                mm[g][0] = __ballot_sync(0xFFFFFFFFu, c0 < 2);
                mm[g][1] = __ballot_sync(0xFFFFFFFFu, c1 < 2);
                uc0 = c0 < uc0 ? c0 : uc0;
                uc1 = c1 < uc1 ? c1 : uc1;
            }
            // union over the heads of the group (with one head it is that head's masks)
            const uint32_t um0 = G == 1 ? mm[0][0] : __ballot_sync(0xFFFFFFFFu, uc0 < 2);
            const uint32_t um1 = G == 1 ? mm[0][1] : __ballot_sync(0xFFFFFFFFu, uc1 < 2);
            const uint32_t bar = bar_full + slot * 8;
            const uint32_t ra = base + pl.rec + slot * REC;
            uint32_t rows = 0, start = 0, nib_bytes = 0, ul0 = 0, ul1 = 0;
            if (um0 | um1) {            // (warp-uniform)
                ul0 = __ballot_sync(0xFFFFFFFFu, uc0 == 0);
                ul1 = __ballot_sync(0xFFFFFFFFu, uc1 == 0);
                rows = __popc(um0) + __popc(um1);
                nib_bytes = (uint32_t)HD * (rows + __popc(ul0) + __popc(ul1));
                // rows of the side ring, taken in token order; wait for older stages to hand theirs back if it is full
                while (alive && side_head + rows - side_tail > (uint32_t)nside) reclaim();
                if (!alive) break;
                start = side_head & (uint32_t)(nside - 1);
                side_head += rows;
            }
            if (lane == 0) {
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(ra), "r"(start), "r"(um0), "r"(um1), "r"(rows) : "memory");
#pragma unroll
                for (int g = 0; g < G; ++g) sts64(ra + 16 + g * 8, mm[g][0], mm[g][1]);
                // publishes the record, announces the nibble bytes; the phase completes when all bytes have landed
                if (nib_bytes) mbar_arrive_expect(bar, nib_bytes);
                else mbar_arrive(bar);
            }
            if (rows) {
                const uint32_t ma = base + pl.mid, la = base + pl.low, wrap = (uint32_t)(nside - 1);
                const size_t src = (size_t)t0 * HD;
                const bool dense = (um0 & um1) == 0xFFFFFFFFu && start + TOK <= (uint32_t)nside;
                if (dense) {
                    // the whole stage reads the mid plane: one 4 KB copy (and one for the low plane when it is all read)
                    if (lane == 0) bulk_copy(ma + start * HD, M + src, TOK * HD, bar);
                    if ((ul0 & ul1) == 0xFFFFFFFFu) {
                        if (lane == 0) bulk_copy(la + start * HD, L + src, TOK * HD, bar);
                    } else {
                        if (uc0 == 0) bulk_copy(la + ((start + lane) & wrap) * HD, L + src + (size_t)lane * HD, HD, bar);
                        if (uc1 == 0) bulk_copy(la + ((start + 32 + lane) & wrap) * HD, L + src + (size_t)(lane + 32) * HD, HD, bar);
                    }
                } else {
                    const uint32_t r0 = (start + __popc(um0 & lt)) & wrap;
                    const uint32_t r1 = (start + __popc(um0) + __popc(um1 & lt)) & wrap;
                    if (uc0 < 2) bulk_copy(ma + r0 * HD, M + src + (size_t)lane * HD, HD, bar);
                    if (uc0 == 0) bulk_copy(la + r0 * HD, L + src + (size_t)lane * HD, HD, bar);
                    if (uc1 < 2) bulk_copy(ma + r1 * HD, M + src + (size_t)(lane + 32) * HD, HD, bar);
                    if (uc1 == 0) bulk_copy(la + r1 * HD, L + src + (size_t)(lane + 32) * HD, HD, bar);
                }
            }
            if (++slot == nf) slot = 0;
            if (++sic == sch) {
                sic = 0;
                ++c;
                if (++cbuf == 3) { cbuf = 0; cpar ^= 1u; }
            }
        }
        // a wait gave up (never expected): give the copies in flight time to land before the CTA's shared memory is
        // released
        if (!alive) for (int k = 0; k < 1000; ++k) __nanosleep(1000);
        if (p.prof && lane == 0) { p.prof[bh * 16 + 10] = clock64() - d_t0; p.prof[bh * 16 + 11] = nslow_free; p.prof[bh * 16 + 12] = nslow_sb; p.prof[bh * 16 + 13] = d_thr; }
        return;
    }

    // ---------------------------------------------------------------------- chain warps
    const int hg = warp >> 1, wh = warp & 1, g0 = hg * HPW;
    const int pair = 32 * wh + 8 * (lane & 3) + (lane >> 2);          // this lane's channel pair
    // ldmatrix row address of this lane inside a group of 8 tokens: matrix lane/8 = tokens 2i, 2i+1; row r of a matrix
    // = token 2i + (r & 1), 16-byte chunk 4*wh + r/2 of the token's row
    const uint32_t lm_off = (uint32_t)((2 * (lane >> 3) + (lane & 1)) * D + (4 * wh + ((lane & 7) >> 1)) * 16);
    uint32_t acc[HPW];
#pragma unroll
    for (int h = 0; h < HPW; ++h) acc[h] = 0;
    bool alive = true;
    const int nsf = n / TOK;                                           // full stages
    uint32_t A[HPW];                                                   // thresholds, for the per-token path

    // Position of a stage in the rings, advanced stage by stage (no divisions in the loop).
    struct Pos {
        int slot;            // ring slot = stage % nf
        uint32_t parity;     // (stage / nf) & 1
        int sic, buf;        // stage inside its probability chunk, chunk % 3
    };
    auto next_pos = [&](Pos q) {
        if (++q.slot == nf) { q.slot = 0; q.parity ^= 1u; }
        if (++q.sic == sch) { q.sic = 0; q.buf = q.buf == 2 ? 0 : q.buf + 1; }
        return q;
    };
    auto f_addr = [&](const Pos& q) { return base + pl.f + (uint32_t)q.slot * F_BYTES; };
    auto s_addr = [&](const Pos& q) {     // probabilities of token 0 of the stage, first head of this warp
        return base + pl.sb + (uint32_t)q.buf * sb_buf + (uint32_t)g0 * sb_head + (uint32_t)q.sic * (TOK * 2);
    };
    auto fetch = [&](VGroup<HPW>& r, uint32_t fa, uint32_t sa, int grp) {
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(r.h[0]), "=r"(r.h[1]), "=r"(r.h[2]), "=r"(r.h[3]) : "r"(fa + (uint32_t)grp * (8 * D) + lm_off));
#pragma unroll
        for (int h = 0; h < HPW; ++h) r.s[h] = lds128(sa + h * sb_head + grp * 16);
    };
    // Low bytes [even channel, odd channel] of this lane's pair for token t of the stage, head h of this warp, from the
    // side ring under the head's own code (V_cache.cu:250-253); 0x8080 when the head reads neither plane.
    auto low_word = [&](const uint4& rec, uint32_t sa, int t, int h) -> uint32_t {
        const uint32_t sb = lds16(sa + h * sb_head + t * 2);
        const int diff = (int)(int16_t)(uint16_t)(A[h] - sb);
        const int code = p.reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
        if (code == 2) return 0x8080u;                                   // (warp-uniform)
        const uint32_t rank = t < 32 ? __popc(rec.y & ((1u << t) - 1u))
                                     : __popc(rec.y) + __popc(rec.z & ((1u << (t - 32)) - 1u));
        const uint32_t row = ((rec.x + rank) & (uint32_t)(nside - 1)) * HD + pair;
        const uint32_t mb = lds8(base + pl.mid + row);
        const uint32_t lb = code == 0 ? lds8(base + pl.low + row) : 0x88u;
        return ((mb & 0xF0u) | (lb >> 4)) | ((((mb & 0x0Fu) << 4) | (lb & 0x0Fu)) << 8);
    };
    // A lean group (no head of this warp reads a nibble plane for any of its 8 tokens): one byte permute per token
    // (high bytes + the constant low byte 0x80) shared by the heads, one FMA per token and head.
    auto lean = [&](const VGroup<HPW>& r) {
        uint32_t k[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) k[u] = __byte_perm(r.h[u >> 1], 0x80808080u, (u & 1) ? 0x3424 : 0x1404);
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int h = 0; h < HPW; ++h) acc[h] = v_fma(k[u], v_dup(u4w(r.s[h], u >> 1), u & 1), acc[h]);
    };
    // Any group: as above, but the k~ words of the flagged tokens (bits of `any`) are patched with the low bytes from
    // the side ring, head by head.  The patch is a short loop over the flagged tokens and exists once: what this path
    // costs is the instruction-cache lines it touches, so it is kept small.
    auto mixed = [&](const VGroup<HPW>& r, const uint4& rec, uint32_t sa, int grp, uint32_t any) {
        uint32_t k[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) k[u] = __byte_perm(r.h[u >> 1], 0x80808080u, (u & 1) ? 0x3424 : 0x1404);
#pragma unroll
        for (int h = 0; h < HPW; ++h) {
            uint32_t kh[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) kh[u] = k[u];
#pragma unroll 1
            for (uint32_t bits = any; bits; bits &= bits - 1) {
                const int u = __ffs(bits) - 1;
                const uint32_t lw = low_word(rec, sa, grp * 8 + u, h);
                const uint32_t hp = (u >> 1) == 0 ? r.h[0] : (u >> 1) == 1 ? r.h[1] : (u >> 1) == 2 ? r.h[2] : r.h[3];
                const uint32_t kk = __byte_perm(hp, lw, (u & 1) ? 0x3524 : 0x1504);
#pragma unroll
                for (int v = 0; v < 8; ++v) kh[v] = (v == u) ? kk : kh[v];
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[h] = v_fma(kh[u], v_dup(u4w(r.s[h], u >> 1), u & 1), acc[h]);
        }
    };
    // Tokens [0, u1) of a partial group, token by token from shared memory (the last few tokens of a sequence whose
    // length is not a multiple of 8).
    auto per_token = [&](const uint4& rec, uint32_t fa, uint32_t sa, int grp, int u1) {
#pragma unroll 1
        for (int u = 0; u < u1; ++u) {
            const int t = grp * 8 + u;
            const uint32_t hw = lds16(fa + (uint32_t)t * D + pair * 2);
#pragma unroll
            for (int h = 0; h < HPW; ++h) {
                const uint32_t sb = lds16(sa + h * sb_head + t * 2);
                acc[h] = hfma2_bits(__byte_perm(hw, low_word(rec, sa, t, h), 0x1504), sb | (sb << 16), acc[h]);
            }
        }
    };
    // this warp's heads' "reads a nibble plane" bits of the stage in ring slot `slot`: lo = tokens 0..31, hi = 32..63
    auto masks = [&](int slot, uint32_t& lo, uint32_t& hi) {
        lo = hi = 0;
#pragma unroll
        for (int h = 0; h < HPW; ++h) {
            const uint2 m = lds64(base + pl.rec + (uint32_t)slot * REC + 16 + (g0 + h) * 8);
            lo |= m.x;
            hi |= m.y;
        }
    };
    auto any_of = [](uint32_t lo, uint32_t hi, int grp) { return ((grp < 4 ? lo : hi) >> ((grp & 3) * 8)) & 0xFFu; };

    VGroup<HPW> ra, rb;
    uint32_t mlo = 0, mhi = 0;
    long long prof_wait = 0, prof_t0 = clock64(), prof_first = 0;
    int nslow_full = 0;
    long long prof_gen = 0;
    Pos cur = {0, 0u, 0, 0};
    uint32_t fa = f_addr(cur), sa = s_addr(cur);
    if (nst > 0) {
        alive = mbar_wait(bar_full, 0);
        prof_first = clock64() - prof_t0;
        if (alive) {
#pragma unroll
            for (int h = 0; h < HPW; ++h) A[h] = lds32(base + pl.thr + (g0 + h) * 4);
            if (nsf > 0) {
                masks(0, mlo, mhi);
                fetch(ra, fa, sa, 0);
            }
        }
    }
    // One full stage per iteration; on entry ra holds group 0 of the stage and (mlo, mhi) its masks.
#pragma unroll 1
    for (int left = nsf; left > 0 && alive; --left) {
        const Pos nxt = next_pos(cur);
        const uint32_t nfa = f_addr(nxt), nsa = s_addr(nxt);
        uint32_t nlo = 0, nhi = 0;
        if (p.dbg & 1) {
            if (left > 1) {
                const long long w0 = clock64();
                alive = mbar_wait(bar_full + nxt.slot * 8, nxt.parity, &nslow_full);
                prof_wait += clock64() - w0;
                if (alive) masks(nxt.slot, nlo, nhi);
            }
        } else if (__builtin_expect((mlo | mhi) == 0, 1)) {
            // lean stage: 64 tokens straight-line, no branch but the wait; groups alternate between ra and rb and the
            // group after next is fetched while one is consumed
#pragma unroll
            for (int ga = 0; ga < 8; ga += 2) {
                fetch(rb, fa, sa, ga + 1);
                lean(ra);
                if (ga < 6) {
                    fetch(ra, fa, sa, ga + 2);
                } else if (left > 1) {
                    // first group of the next stage; it has normally landed long ago (the ring is several stages deep)
                    const long long w0 = clock64();
                    alive = mbar_wait(bar_full + nxt.slot * 8, nxt.parity, &nslow_full);
                    prof_wait += clock64() - w0;
                    if (alive) {
                        masks(nxt.slot, nlo, nhi);
                        fetch(ra, nfa, nsa, 0);
                    }
                }
                lean(rb);
            }
        } else {
            // a stage in which some token reads a nibble plane: one group per iteration through one copy of compact code
            const long long g0c = clock64();
            const uint4 rec = lds128(base + pl.rec + (uint32_t)cur.slot * REC);   // {first side row, union lo, hi, rows}
#pragma unroll 1
            for (int grp = 0; grp < 8; ++grp) {
                if (grp > 0) fetch(ra, fa, sa, grp);
                mixed(ra, rec, sa, grp, any_of(mlo, mhi, grp));
            }
            if (left > 1) {
                alive = mbar_wait(bar_full + nxt.slot * 8, nxt.parity, &nslow_full);
                if (alive) {
                    masks(nxt.slot, nlo, nhi);
                    fetch(ra, nfa, nsa, 0);
                }
            }
            prof_gen += clock64() - g0c;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_free + cur.slot * 8);           // ring slot, side rows and record are free
        cur = nxt; fa = nfa; sa = nsa; mlo = nlo; mhi = nhi;
    }
    const int tail = n - nsf * TOK;
    if (tail > 0 && alive) {
        // last, partial stage (rows of the slot beyond the last token hold stale bytes that are never used)
        if (nsf > 0) alive = mbar_wait(bar_full + cur.slot * 8, cur.parity);
        if (alive) {
            masks(cur.slot, mlo, mhi);
            const uint4 rec = lds128(base + pl.rec + (uint32_t)cur.slot * REC);
            for (int grp = 0; grp * 8 < tail; ++grp) {
                const int u1 = tail - grp * 8 < 8 ? tail - grp * 8 : 8;
                if (u1 == 8) {
                    fetch(ra, fa, sa, grp);
                    mixed(ra, rec, sa, grp, any_of(mlo, mhi, grp));
                } else {
                    per_token(rec, fa, sa, grp, u1);
                }
            }
        }
    }
    if (p.prof && lane == 0) {
        const long long t1 = clock64();
        p.prof[bh * 16 + warp] = t1 - prof_t0;
        p.prof[bh * 16 + 4 + warp] = prof_wait;
        if (warp == 0) { p.prof[bh * 16 + 14] = nslow_full; p.prof[bh * 16 + 7] = prof_gen; }
        if (warp == 0) { p.prof[bh * 16 + 2] = prof_first; }
    }
#pragma unroll
    for (int h = 0; h < HPW; ++h)
        reinterpret_cast<uint32_t*>(p.o)[((size_t)bh * G + g0 + h) * 64 + pair] = alive ? acc[h] : 0x7E007E00u;
}

}  // namespace akv
