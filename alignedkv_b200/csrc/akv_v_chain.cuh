// Exact-order P.V, streaming form for multi-head attention: the kernel body behind v_cache_compute for head_dim 128.
//
// Replaces the reference's v_cache_compute_kernel (extension/csrc/V_cache.cu:178-308); bit-identical outputs: every
// output channel is the fp16 fused-multiply-add chain over tokens 0..n-1 in order (V_cache.cu:203,304), skipped nibble
// planes are replaced by the reference's constants (V_cache.cu:198-202,250-253).
//
// Design (B200).  The token order leaves one dependent chain per (batch, head, channel pair), and the V layout is
// token-major (a token's 128 high bytes are one row) while a chain thread wants "my channel pairs, next tokens".  That
// transposition is done by the load instruction: ldmatrix.x4.trans over four token rows (one 8x8 matrix of 16-bit
// words per token: its eight 16-byte chunks, 128 contiguous bytes, so no bank conflict) hands lane T, for each of
// the four tokens, one register holding the high-byte pairs of channel pairs 16*(T%4) + T/4 and 16*(T%4) + 8 + T/4.
// The LOW bytes come the same way from a table of the same shape that holds 0x80 for every channel of every token
// (the reference's substitute when neither nibble plane is read: the rule, in aligned mode) except for the few tokens
// whose probability lies within two binades of the threshold; their rows are built from the nibble planes.  So the
// chain warp runs ONE branch-free instruction stream for every token: per 8 tokens four ldmatrix and one 16-byte load
// of probabilities, per token two byte permutes (high + low bytes -> two fp16 pairs) and two FMAs - two independent
// chains per thread, which hide the FMA latency.  That matters more than it seems: a warp whose steady loop carries
// branches and rarely-run code, or does not fit the scheduler's instruction cache, was measured at a third of the
// speed of the same arithmetic in a straight line.
//   A unit = one (batch, query head).  A CTA holds UPC rings of high bytes; a ring serves GH heads - one, or the query
//   heads of one KV head, which need the same high bytes - and every head has its own chain warp, decision warps,
//   tables and barriers.  (With a ring per query head the heads of a KV head are neighbouring units that stream the same
//   planes at the same pace: the first one's copies bring a stage into L2, the others' hit there.)
//   chain warp: all 64 channel pairs of the head, one 64-token stage per loop iteration.
//   copy warp (one per ring): stage i -> ring slot i % nf as soon as every chain of the ring has released the slot's
//     previous stage: one 8 KB bulk asynchronous copy of the high bytes exactly as they lie in the plane.
//   decision warps (NDW per head, stage i belongs to warp i % NDW): lane = tokens (lane, lane + 32) of a stage.  EARLY
//     part, a ring ahead of its use: takes the probabilities from a buffer bulk-copied a chunk ahead, decides the read
//     codes (V_cache.cu:211,250-251), reserves rows of a small side ring for the tokens that read a nibble plane and
//     starts 64-byte copies of just those rows (one 4 KB copy when the whole stage reads a plane), counted on a barrier
//     of their own.  LATE part, when the stage's ring slot is free: restores the table rows the slot's previous stage
//     had patched, makes sure the nibble rows have landed (long ago), builds the flagged tokens' rows of the low-byte
//     table, and arrives on the stage's barrier.  Requesting the nibble rows a ring ahead matters: issued together with
//     the stage's high bytes, the few small copies completed late under load and held up every stage that had one.
//     And the NUMBER of these warps matters: a stage with flagged tokens costs its warp three out-of-line calls, and
//     two warps per head fell behind the chain on every such stage (34.9 us for batch 8 x 32 heads x 4096 tokens);
//     four, on schedulers the chain warps do not use, keep up (28.5 us, with or without flagged tokens).
// Every wait is bounded (about a second); a wait that runs out raises the device error flag, the chain stores NaN
// instead of a result, and the producers give their copies in flight time to land before the CTA leaves.
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
    int npt;                // streaming form: low-byte tables per head (even: half of them per decision warp)
    int units;              // streaming form: number of ring units (heads / heads per ring)
    // streaming form: res != nullptr adds the residual tokens' part of the output, [B, Hq, D] fp16 computed by the
    // softmax kernel: out = half(o + res) (extension/v_cache_file.py:189), which saves the tail launch
    const uint16_t* res;
};

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
// Non-blocking: has the phase with this parity completed?
__device__ __forceinline__ uint32_t mbar_test(uint32_t a, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ bool mbar_wait(uint32_t a, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    if (__builtin_expect(ok != 0, 1)) return true;
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
constexpr int F_BYTES = TOK * D;   // high bytes of a stage (and its rows of the low-byte table)
constexpr int REC = 16;            // record of a stage: {first side row, flagged tokens 0..31, 32..63, rows | (table + 1) << 8}

// Shared-memory plan of a CTA (byte offsets), computed the same way on both sides.  A CTA holds `upc` rings, each
// shared by `gh` heads (gh > 1: the query heads of one KV head read the same high bytes).
struct Plan {
    int ctab;                        // the constant low-byte table (0x80 everywhere), one per CTA
    int ring0, ring_bytes, rbar;     // ring r at ring0 + r * ring_bytes: nf stages of high bytes, then full[nf], free[nf] at rbar
    int head0, head_bytes;           // head u at head0 + u * head_bytes, inside it:
    int lw, mid, low, sb, rec, thr, bar;
    int bytes;
};
__host__ __device__ inline Plan plan(int nf, int nside, int sch, int npt, int upc, int gh) {
    Plan p;
    p.ctab = 0;
    p.ring0 = F_BYTES;
    p.rbar = nf * F_BYTES;
    p.ring_bytes = (nf * F_BYTES + 2 * nf * 8 + 127) & ~127;
    p.head0 = p.ring0 + upc * p.ring_bytes;
    p.lw = 0;                                  // npt low-byte tables, each of a stage's shape
    p.mid = npt * F_BYTES;                     // side rings: rows of the mid / low nibble planes
    p.low = p.mid + nside * HD;
    p.sb = p.low + nside * HD;                 // three probability buffers of sch x 64 values
    p.rec = p.sb + 3 * sch * TOK * 2;          // 2 nf records
    p.thr = p.rec + 2 * nf * REC;              // threshold (already shifted)
    p.bar = (p.thr + 4 + 7) & ~7;              // probability buffers[3], nibble rows[2 nf]
    p.head_bytes = (p.bar + (2 * nf + 3) * 8 + 127) & ~127;
    p.bytes = p.head0 + upc * gh * p.head_bytes;
    return p;
}
}  // namespace vch

// Both halves of the result = half `hi ? 1 : 0` of w (the probability of one token for both channels of a pair).
__device__ __forceinline__ __half2 v_dup(uint32_t w, int hi) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    return hi ? __high2half2(h) : __low2half2(h);
}
__device__ __forceinline__ uint32_t v_fma(uint32_t k, __half2 s, uint32_t acc) {
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&k), s, *reinterpret_cast<const __half2*>(&acc));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// About a millisecond of sleep: after a wait gave up (never expected), the copies in flight get time to land before
// the CTA's shared memory is released.
__device__ __noinline__ void v_sleep_ms() {
#pragma unroll 1
    for (int k = 0; k < 1000; ++k) __nanosleep(1000);
}

// Starts the copies of the nibble rows of one stage into the side ring and announces their bytes on `bar` (one
// arrival).  Out of line: it runs for the minority of stages in which some token reads a nibble plane, and the
// decision warp's steady loop has to stay small.
//   M, L: mid / low plane rows of the stage's token 0;  ma, la: side rings;  start: first side row;  wrap: rows - 1
//   um0 / um1: tokens 0..31 / 32..63 that read the mid plane;  c0 / c1: this lane's codes of tokens lane / lane+32
__device__ __noinline__ void v_issue_nibble_rows(const uint8_t* M, const uint8_t* L, uint32_t ma, uint32_t la, uint32_t bar,
                                                 uint32_t start, uint32_t wrap, uint32_t um0, uint32_t um1, int c0, int c1,
                                                 int lane) {
    using namespace vch;
    const uint32_t ul0 = __ballot_sync(0xFFFFFFFFu, c0 == 0), ul1 = __ballot_sync(0xFFFFFFFFu, c1 == 0);
    const uint32_t rows = __popc(um0) + __popc(um1);
    if (lane == 0) mbar_arrive_expect(bar, (uint32_t)HD * (rows + __popc(ul0) + __popc(ul1)));
    __syncwarp();
    const uint32_t lt = (1u << lane) - 1u;
    if ((um0 & um1) == 0xFFFFFFFFu && start + TOK <= wrap + 1) {
        // the whole stage reads the mid plane: one 4 KB copy (and one for the low plane when it is all read)
        if (lane == 0) bulk_copy(ma + start * HD, M, TOK * HD, bar);
        if ((ul0 & ul1) == 0xFFFFFFFFu) {
            if (lane == 0) bulk_copy(la + start * HD, L, TOK * HD, bar);
        } else {
            if (c0 == 0) bulk_copy(la + ((start + lane) & wrap) * HD, L + (size_t)lane * HD, HD, bar);
            if (c1 == 0) bulk_copy(la + ((start + 32 + lane) & wrap) * HD, L + (size_t)(lane + 32) * HD, HD, bar);
        }
    } else {
        const uint32_t r0 = (start + __popc(um0 & lt)) & wrap;
        const uint32_t r1 = (start + __popc(um0) + __popc(um1 & lt)) & wrap;
        if (c0 < 2) bulk_copy(ma + r0 * HD, M + (size_t)lane * HD, HD, bar);
        if (c0 == 0) bulk_copy(la + r0 * HD, L + (size_t)lane * HD, HD, bar);
        if (c1 < 2) bulk_copy(ma + r1 * HD, M + (size_t)(lane + 32) * HD, HD, bar);
        if (c1 == 0) bulk_copy(la + r1 * HD, L + (size_t)(lane + 32) * HD, HD, bar);
    }
}

// Builds the rows of the low-byte table for the flagged tokens of one stage from the side ring (V_cache.cu:250-253):
// channel pair p of a token has mid byte [even channel nibble | odd channel nibble] and low byte likewise; the low
// byte of the even channel is (mid & 0xF0) | (low >> 4), of the odd one ((mid & 0x0F) << 4) | (low & 0x0F); a token
// that reads only the mid plane takes 0x88 for the low-plane byte.  Lane l builds channel pairs 2l, 2l+1 (4 bytes).
//   lw: the stage's rows of the table;  ma, la: side rings;  rec: {first side row, flagged 0..31, 32..63, rows}
//   s_a: the stage's probabilities;  thr: shifted threshold
__device__ __noinline__ void v_build_low_rows(uint32_t lw, uint32_t ma, uint32_t la, uint4 rec, uint32_t wrap, uint32_t s_a,
                                              uint32_t thr, int reference, int lane) {
    using namespace vch;
    uint32_t rank = 0;
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
#pragma unroll 1
        for (uint32_t bits = half ? rec.z : rec.y; bits; bits &= bits - 1, ++rank) {
            const int t = half * 32 + __ffs(bits) - 1;
            const uint32_t sb = lds16(s_a + t * 2);
            const int diff = (int)(int16_t)(uint16_t)(thr - sb);
            const bool low_too = reference || diff < 0x0400;             // (the token reads the mid plane: it is flagged)
            const uint32_t row = ((rec.x + rank) & wrap) * HD + 2 * lane;
            const uint32_t mb = lds16(ma + row);                          // pairs 2l, 2l+1
            const uint32_t lb = low_too ? lds16(la + row) : 0x8888u;
            const uint32_t even = (mb & 0xF0F0u) | ((lb >> 4) & 0x0F0Fu);     // [pair 2l, pair 2l+1] even channels
            const uint32_t odd = ((mb & 0x0F0Fu) << 4) | (lb & 0x0F0Fu);
            // bytes: [even(2l), odd(2l), even(2l+1), odd(2l+1)]
            const uint32_t w = (even & 0xFFu) | ((odd & 0xFFu) << 8) | ((even & 0xFF00u) << 8) | ((odd & 0xFF00u) << 16);
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(lw + (uint32_t)t * D + lane * 4), "r"(w) : "memory");
        }
    }
}

// Puts the constant 0x80 back into the table rows of the tokens flagged in (m0, m1).
__device__ __noinline__ void v_restore_low_rows(uint32_t lw, uint32_t m0, uint32_t m1, int lane) {
    using namespace vch;
#pragma unroll 1
    for (int half = 0; half < 2; ++half)
#pragma unroll 1
        for (uint32_t bits = half ? m1 : m0; bits; bits &= bits - 1)
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(lw + (uint32_t)(half * 32 + __ffs(bits) - 1) * D + lane * 4),
                         "r"(0x80808080u) : "memory");
}

// UPC rings per CTA, GH heads per ring, NDW decision warps per head (2, or 4 with two rings of one head each).
template <int UPC, int GH, int NDW>
__global__ void __launch_bounds__(NDW == 2 ? ((1 + NDW) * UPC * GH + UPC) * 32 : 512, 1) v_chain_kernel(const VParams p) {
    static_assert(NDW == 2 || (NDW == 4 && UPC == 2 && GH == 1), "decision warps per head");
    using namespace vch;
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NU = UPC * GH;                   // heads of the CTA
    // Low-byte tables.  One head per ring: a table per ring slot (npt == nf), patched for the slot's stage and restored
    // when the slot is released - a stage without flagged tokens finds the constant there, and the chain needs neither
    // the record nor a select.  Several heads per ring: there is no room for that, so each decision warp has a few
    // tables it hands to its stages with flagged tokens, and the other stages read the CTA's constant table.
    constexpr bool SLOT_TABLES = GH == 1;
    const int tid = threadIdx.x, lane = tid & 31, wcta = tid >> 5;
    // Warp roles: per head a chain warp and two decision warps (even / odd stages: one warp's serial walk through a
    // stage takes longer than the chain needs to consume it), per ring a copy warp.  Order in the CTA: the chain warps,
    // the even-stage decision warps, the copy warps, the odd-stage decision warps.  The warps are spread over the SM's
    // four schedulers by index, so with two rings of one head each chain warp shares its scheduler only with its copy
    // warp (a handful of instructions per stage) and the four decision warps have the other two; with four heads on
    // one ring every scheduler has one chain warp.
    int role, hu, dw = 0;                          // 0: chain, 1: decision (warp dw of its head), 3: copy, -1: none; head of the CTA
    if (NDW == 2) {
        if (wcta < NU) { role = 0; hu = wcta; }
        else if (wcta < 2 * NU) { role = 1; hu = wcta - NU; }
        else if (wcta < 2 * NU + UPC) { role = 3; hu = (wcta - 2 * NU) * GH; }
        else { role = 1; dw = 1; hu = wcta - 2 * NU - UPC; }
    } else {
        // sixteen warps in groups of four (one per scheduler): schedulers 0, 1 get [chain, copy, -, -] of ring 0 / 1,
        // schedulers 2, 3 the four decision warps of head 0 / 1 - a chain warp never shares its scheduler with a
        // decision warp, whose bursts of work would take issue slots from it
        const int q4 = wcta >> 2, r4 = wcta & 3;
        if (r4 < 2) { hu = r4; role = q4 == 0 ? 0 : (q4 == 1 ? 3 : -1); }
        else { hu = r4 - 2; role = 1; dw = q4; }
    }
    const int ring = hu / GH, hg = hu - ring * GH;
    const long long ru = (long long)blockIdx.x * UPC + ring;   // ring unit
    const long long bh = ru * GH + hg;                         // (batch, query head)
    const long long kv = (ru * GH) / p.group;                  // (batch, KV head) whose planes the ring streams
    const int n = p.n, nf = p.nf, nside = p.nside, sch = p.sch;
    const int nst = (n + TOK - 1) / TOK;
    const Plan pl = plan(nf, nside, sch, p.npt, UPC, GH);
    const uint32_t cta = smem_u32(smem);
    const uint32_t rbase = cta + pl.ring0 + (uint32_t)ring * pl.ring_bytes;    // the ring's stages of high bytes
    const uint32_t base = cta + pl.head0 + (uint32_t)hu * pl.head_bytes;       // everything of this head
    const uint32_t bar_full = rbase + pl.rbar, bar_free = bar_full + nf * 8;
    const uint32_t bar_sb = base + pl.bar, bar_nib = bar_sb + 3 * 8;
    const uint32_t ctab = cta + pl.ctab;

    pdl_enter();
    if (!SLOT_TABLES)
        for (int i = tid; i < F_BYTES / 16; i += blockDim.x)
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(ctab + i * 16), "r"(0x80808080u) : "memory");
    if (role == 0) {
        if (lane == 0) {
            if (hg == 0)
                for (int s = 0; s < nf; ++s) {
                    mbar_init(bar_full + s * 8, 1 + GH);   // the copy warp's arrival (+ the high bytes) and one decision warp's per head
                    mbar_init(bar_free + s * 8, GH);       // the chain warps' arrivals
                }
            for (int s = 0; s < 3; ++s) mbar_init(bar_sb + s * 8, 1);
            for (int s = 0; s < 2 * nf; ++s) mbar_init(bar_nib + s * 8, 1);
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        // the head's own low-byte tables start as the constant too: 0x80 for every channel of every token
        for (int i = lane; i < p.npt * F_BYTES / 16; i += 32)
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(base + pl.lw + i * 16), "r"(0x80808080u) : "memory");
    }
    __syncthreads();
    if (role < 0 || ru >= p.units) return;         // (odd number of ring units: the last CTA's second ring has none)

    if (role == 3) {
        // ------------------------------------------------------------------ copy warp: the high bytes
        const uint8_t* F = p.first8 + (size_t)kv * p.max_seq_len * D;
        int slot = 0;
        uint32_t parity = 0;                       // of the release being waited for: (i / nf - 1) & 1
        bool alive = true;
        // The decision warp's first loads (probe result, exponent maxima) go out before this warp floods the memory
        // system with the first ring of copies - behind that flood they would take several times as long, and the
        // first stage cannot be consumed before the threshold is known.
        asm volatile("bar.sync %0, %1;\n" ::"r"(1 + ring), "r"((NDW * GH + 1) * 32) : "memory");
#pragma unroll 1
        for (int i = 0; i < nst; ++i) {
            if (i >= nf) {
                alive = mbar_wait(bar_free + slot * 8, parity);
                if (!alive) break;
            }
            if (lane == 0) {
                const int cnt = (n - i * TOK) < TOK ? (n - i * TOK) : TOK;
                const uint32_t bar = bar_full + slot * 8;
                mbar_arrive_expect(bar, (uint32_t)cnt * D);
                bulk_copy(rbase + (uint32_t)slot * F_BYTES, F + (size_t)i * TOK * D, (uint32_t)cnt * D, bar);
            }
            if (++slot == nf) { slot = 0; if (i >= nf) parity ^= 1u; }
        }
        if (!alive) v_sleep_ms();
        return;
    }
    if (role == 1) {
        // ------------------------------------------------------------------ decision warps
        // Warp w (0 .. NDW-1) owns the stages i with i % NDW == w.  The ring depth nf is a multiple of NDW, so the
        // previous stage of a ring slot belongs to the same warp, and each warp has its own part of the side ring: the
        // warps never share state.
        const int w = dw;
        const uint8_t* M = p.mid4 + (size_t)kv * p.max_seq_len * HD;
        const uint8_t* L = p.last4 + (size_t)kv * p.max_seq_len * HD;
        const uint16_t* s_row = p.s + (size_t)bh * p.s_last_dim;
        bool alive = true;
        // probability chunk c (stages c*sch ..) -> buffer `buf` = c % 3; issued by one thread of warp 0
        auto request_s = [&](int c, int buf) {
            const int t0 = c * sch * TOK;
            int cnt = n - t0;
            cnt = cnt > sch * TOK ? sch * TOK : cnt;
            const uint32_t bytes = (uint32_t)((cnt + 7) & ~7) * 2;     // rows are padded to a multiple of 8 values
            mbar_arrive_expect(bar_sb + buf * 8, bytes);
            bulk_copy(base + pl.sb + (uint32_t)buf * (sch * TOK * 2), s_row + t0, bytes, bar_sb + buf * 8);
        };
        if (w == 0 && lane == 0 && nst > 0) request_s(0, 0);
        // threshold: from the probe result (decode step) or as given
        uint32_t a;
        if (p.test_o) {
            a = v_threshold_warp(p.test_o, p.v_exp, bh, p.H, p.group, D, lane);
            if (w == 0 && lane == 0) p.amin_out[bh] = (uint8_t)a;
        } else {
            a = p.amin[bh];
        }
        const uint32_t A = (a << 10) & 0xFFFFu;
        asm volatile("bar.sync %0, %1;\n" ::"r"(1 + ring), "r"((NDW * GH + 1) * 32) : "memory");
        const int hside = nside / NDW;                     // rows of this warp's part of the side ring
        const uint32_t ma = base + pl.mid + (uint32_t)w * hside * HD, la = base + pl.low + (uint32_t)w * hside * HD;
        const uint32_t wrap = (uint32_t)(hside - 1);
        uint32_t side_head = 0, side_tail = 0;    // side rows handed out / taken back so far
        const int nrec = 2 * nf;
        int freed = w, freed_slot = w, freed_rec = w;   // next own stage whose release is to be consumed; % nf, % 2nf
        uint32_t freed_parity = 0;                      // (freed / nf) & 1
        uint32_t nib_par = 0;                           // bit r: parity of the NEXT phase of nibble barrier r
        // low-byte tables of this warp, used in turn by its stages with flagged tokens; t_out = tables in use (built
        // and not yet restored)
        const int npw = p.npt / NDW;
        int t_next = 0, t_out = 0;
        // consume the release of own stage `freed`: its side rows are free again, its patched table rows become 0x80 again
        auto reclaim = [&]() {
            alive = mbar_wait(bar_free + freed_slot * 8, freed_parity);
            const uint4 rec = lds128(base + pl.rec + freed_rec * REC);
            if (__builtin_expect(rec.w != 0, 0)) {
                side_tail += rec.w & 0xFFu;
                if (alive && (rec.w >> 8) != 0) {           // (a stage that was prepared but never armed has no table)
                    v_restore_low_rows(base + pl.lw + ((rec.w >> 8) - 1u) * F_BYTES, rec.y, rec.z, lane);
                    --t_out;
                }
            }
            freed += NDW;
            if ((freed_slot += NDW) >= nf) { freed_slot -= nf; freed_parity ^= 1u; }
            if ((freed_rec += NDW) >= nrec) freed_rec -= nrec;
        };
        // EARLY part for own stage j (position state advances with j).  armed = next own stage to be armed: side rows
        // can only be waited for while an armed own stage is still unreleased; otherwise the stage is prepared later
        // (returns false).
        int e_rec = w, e_sic = w, e_c = 0, e_buf = 0;   // of stage j: j % 2nf, j % sch, j / sch, (j / sch) % 3
        uint32_t e_par = 0;                             // ((j / sch) / 3) & 1
        bool e_chunk = false;                           // the chunk of stage j has been entered
        auto early = [&](int j, int armed) -> bool {
            if (e_sic < NDW && !e_chunk) {    // entering chunk c: ask for the next one (warp 0), make sure this one has landed
                if (w == 0 && (e_c + 1) * sch < nst && lane == 0) request_s(e_c + 1, e_buf == 2 ? 0 : e_buf + 1);
                alive = mbar_wait(bar_sb + e_buf * 8, e_par);
                if (!alive) return false;
                e_chunk = true;
            }
            const int t0 = j * TOK;
            const int cnt = (n - t0) < TOK ? (n - t0) : TOK;
            // read codes of tokens `lane` and `lane + 32` from the bit patterns (V_cache.cu:211,250-251): 16-bit
            // wrap-around, signed compare  (beyond the last token the buffer holds stale but readable bytes)
            const uint32_t sa = base + pl.sb + (uint32_t)e_buf * (sch * TOK * 2) + (uint32_t)e_sic * (TOK * 2) + lane * 2;
            const uint32_t s0 = lds16(sa), s1 = lds16(sa + 64);
            const int d0 = (int)(int16_t)(uint16_t)(A - s0), d1 = (int)(int16_t)(uint16_t)(A - s1);
            int c0 = p.reference ? 0 : (d0 >= 0x0800 ? 2 : (d0 >= 0x0400 ? 1 : 0));
            int c1 = p.reference ? 0 : (d1 >= 0x0800 ? 2 : (d1 >= 0x0400 ? 1 : 0));
            if (lane >= cnt) c0 = 2;
            if (lane + 32 >= cnt) c1 = 2;
            const uint32_t um0 = __ballot_sync(0xFFFFFFFFu, c0 < 2), um1 = __ballot_sync(0xFFFFFFFFu, c1 < 2);
            uint32_t rows = 0, start = 0;
            if (__builtin_expect((um0 | um1) != 0, 0)) {    // (warp-uniform)
                rows = __popc(um0) + __popc(um1);
                // rows of the side ring, taken in token order; wait for older stages to hand theirs back if it is full
                while (alive && side_head + rows - side_tail > (uint32_t)hside) {
                    if (freed >= armed) return false;       // nothing armed is outstanding: prepare this stage later
                    reclaim();
                }
                if (!alive) return false;
                start = side_head & wrap;
                side_head += rows;
                nib_par ^= 1u << e_rec;
                v_issue_nibble_rows(M + (size_t)t0 * HD, L + (size_t)t0 * HD, ma, la, bar_nib + e_rec * 8, start, wrap, um0,
                                    um1, c0, c1, lane);
            }
            if (lane == 0)
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(base + pl.rec + e_rec * REC), "r"(start), "r"(um0),
                             "r"(um1), "r"(rows) : "memory");
            __syncwarp();               // (the record is read back by every lane in the late part)
            if ((e_rec += NDW) >= nrec) e_rec -= nrec;
            e_chunk = false;
            if ((e_sic += NDW) >= sch) {
                e_sic -= sch;
                ++e_c;
                if (++e_buf == 3) { e_buf = 0; e_par ^= 1u; }
            }
            return true;
        };
        int slot = w, rec = w, j = w;             // of stage i: i % nf, i % 2nf; j: next own stage to prepare
        int l_sic = w, l_buf = 0;                 // of stage i: i % sch, (i / sch) % 3
#pragma unroll 1
        for (int i = w; i < nst && alive; i += NDW) {
            while (alive && freed <= i - nf) reclaim();
            // phase 0: stage i must be prepared (it normally is, a ring ago), then it is armed; phase 1: run ahead, up
            // to a ring's length (one call site of the early part for both)
#pragma unroll 1
            for (int phase = 0; phase < 2 && alive; ++phase) {
                const int lim = phase == 0 ? i : i + nf;
#pragma unroll 1
                while (alive && j <= lim && j < nst) {
                    if (!early(j, i + NDW * phase)) break;
                    j += NDW;
                }
                if (phase == 0 && alive) {
                    // LATE part of stage i: its nibble rows (requested long ago) must have landed and its rows of the
                    // low-byte table be built; then it is armed
                    const uint4 r = lds128(base + pl.rec + rec * REC);
                    if (__builtin_expect(r.w != 0, 0)) {
                        // a table of this warp: the oldest one in use is handed back when its (armed) stage is released
                        while (!SLOT_TABLES && alive && t_out >= npw) reclaim();
                        if (alive) alive = mbar_wait(bar_nib + rec * 8, ((nib_par >> rec) & 1u) ^ 1u);
                        if (alive) {
                            const uint32_t tbl = SLOT_TABLES ? (uint32_t)slot : (uint32_t)(w * npw + t_next);
                            v_build_low_rows(base + pl.lw + tbl * F_BYTES, ma, la, r, wrap,
                                             base + pl.sb + (uint32_t)l_buf * (sch * TOK * 2) + (uint32_t)l_sic * (TOK * 2), A,
                                             p.reference, lane);
                            if (lane == 0)
                                asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(base + pl.rec + rec * REC + 12),
                                             "r"(r.w | ((tbl + 1u) << 8)) : "memory");
                            t_next = t_next + 1 == npw ? 0 : t_next + 1;
                            ++t_out;
                        }
                    }
                    __syncwarp();
                    if (lane == 0 && alive) mbar_arrive(bar_full + slot * 8);   // publishes the table rows; the copy warp adds the bytes
                    if ((slot += NDW) >= nf) slot -= nf;
                    if ((rec += NDW) >= nrec) rec -= nrec;
                    if ((l_sic += NDW) >= sch) { l_sic -= sch; l_buf = l_buf == 2 ? 0 : l_buf + 1; }
                }
            }
        }
        if (!alive) v_sleep_ms();
        return;
    }

    // ---------------------------------------------------------------------- chain warp
    const int pairA = 16 * (lane & 3) + (lane >> 2), pairB = pairA + 8;   // this lane's channel pairs
    // ldmatrix row address of this lane inside four token rows: matrix lane/8 = token, row lane%8 = 16-byte chunk
    const uint32_t lm_off = (uint32_t)((lane >> 3) * D + (lane & 7) * 16);
    uint32_t accA = 0, accB = 0;
    bool alive = true;
    const int nsf = n / TOK;                                           // full stages
    const int nrec = 2 * nf;                                           // records: one per stage, a ring of two ring lengths
    // Registers of one group of 8 tokens: per token [pair A even, odd | pair B even, odd] high bytes and low bytes, and
    // the 8 probabilities.
    struct Grp {
        uint32_t h[8], l[8];
        uint4 s;
    };
    auto ldm = [](uint32_t (&r)[8], int o, uint32_t a) {
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(r[o]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]) : "r"(a));
    };
    // A stage without flagged tokens (most of them) has the constant low byte 0x80 everywhere: it is consumed by a
    // second copy of the stage body that neither loads the table nor holds its words (LEAN).  la: the low-byte table of
    // a stage WITH flagged tokens (0 for the others): the table of its ring slot, or one of the head's own tables.
    auto fetch_high = [&](Grp& r, uint32_t fa, uint32_t sa, int grp) {
        const uint32_t a = (uint32_t)grp * (8 * D) + lm_off;
        ldm(r.h, 0, fa + a);
        ldm(r.h, 4, fa + a + 4 * D);
        r.s = lds128(sa + grp * 16);
    };
    auto fetch_low = [&](Grp& r, uint32_t la, int grp) {
        const uint32_t a = (uint32_t)grp * (8 * D) + lm_off;
        ldm(r.l, 0, la + a);
        ldm(r.l, 4, la + a + 4 * D);
    };
    auto consume = [&](const Grp& r, auto lean) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const __half2 sd = v_dup(u4w(r.s, u >> 1), u & 1);
            if (decltype(lean)::value) {
                accA = v_fma(__byte_perm(r.h[u], 0x80808080u, 0x1404), sd, accA);
                accB = v_fma(__byte_perm(r.h[u], 0x80808080u, 0x3424), sd, accB);
            } else {
                accA = v_fma(__byte_perm(r.h[u], r.l[u], 0x1504), sd, accA);
                accB = v_fma(__byte_perm(r.h[u], r.l[u], 0x3726), sd, accB);
            }
        }
    };
    int slot = 0, sic = 0, buf = 0, crec = 0;                          // of the current stage: % nf, % sch, chunk % 3, % 2 nf
    uint32_t parity = 0;
    auto f_addr = [&]() { return rbase + (uint32_t)slot * F_BYTES; };
    auto s_addr = [&]() { return base + pl.sb + (uint32_t)buf * (sch * TOK * 2) + (uint32_t)sic * (TOK * 2); };
    // the stage's table: the one of its ring slot (which holds the constant for a stage without flagged tokens, so
    // that form runs one copy of the stage body only: the second copy costs it more in instruction fetch than the
    // skipped loads save - 31.8 against 29.0 us), or from its record (word 3: flagged rows | (table + 1) << 8;
    // 0 = no flagged token -> 0)
    auto l_addr = [&]() -> uint32_t {
        if (SLOT_TABLES) return base + pl.lw + (uint32_t)slot * F_BYTES;
        const uint32_t w = lds32(base + pl.rec + (uint32_t)crec * REC + 12);
        return w ? base + pl.lw + ((w >> 8) - 1u) * F_BYTES : 0u;
    };
    Grp ra, rb;
    uint32_t fa = f_addr(), sa = s_addr(), la = 0;
    if (nst > 0) {
        alive = mbar_wait(bar_full, 0);
        if (alive) la = l_addr();
        if (alive && nsf > 0) {
            fetch_high(ra, fa, sa, 0);
            if (la) fetch_low(ra, la, 0);
        }
    }
    // One full stage per iteration, straight-line: groups alternate between ra and rb, the group after next is
    // fetched while one is consumed; on entry ra holds group 0 of the stage.
#pragma unroll 1
    for (int left = nsf; left > 0 && alive; --left) {
        const int cslot = slot;
        if (++slot == nf) { slot = 0; parity ^= 1u; }
        if (++sic == sch) { sic = 0; buf = buf == 2 ? 0 : buf + 1; }
        if (++crec == nrec) crec = 0;
        const uint32_t nfa = f_addr(), nsa = s_addr();
        uint32_t nla = 0;
        auto stage = [&](auto lean) {
            uint32_t landed = 0;
#pragma unroll
            for (int ga = 0; ga < 8; ga += 2) {
                fetch_high(rb, fa, sa, ga + 1);
                if (!decltype(lean)::value) fetch_low(rb, la, ga + 1);
                consume(ra, lean);
                if (ga < 6) {
                    fetch_high(ra, fa, sa, ga + 2);
                    if (!decltype(lean)::value) fetch_low(ra, la, ga + 2);
                    // the next stage has normally landed long ago (the ring is several stages deep): probe its barrier
                    // two groups before the answer is needed, so that the probe's latency is hidden; then its record
                    if (ga == 2 && left > 1) landed = mbar_test(bar_full + slot * 8, parity);
                    if (ga == 4 && left > 1) nla = l_addr();          // (valid only if it had landed)
                } else if (left > 1) {
                    if (__builtin_expect(!landed, 0)) {
                        alive = mbar_wait(bar_full + slot * 8, parity);
                        nla = l_addr();
                    }
                    if (alive) {                                      // first group of the next stage
                        fetch_high(ra, nfa, nsa, 0);
                        if (nla) fetch_low(ra, nla, 0);
                    }
                }
                consume(rb, lean);
            }
        };
        if constexpr (SLOT_TABLES) {
            stage(std::false_type{});               // (the only copy of the stage body in this instantiation)
        } else {
            if (la) stage(std::false_type{});
            else stage(std::true_type{});
        }
        // the stage is consumed: hand back its ring slot
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_free + cslot * 8);
        fa = nfa; sa = nsa; la = nla;
    }
    const int tail = n - nsf * TOK;
    if (tail > 0 && alive) {
        // last, partial stage, token by token (rows of the slot beyond the last token hold stale bytes, never used)
        if (nsf > 0) alive = mbar_wait(bar_full + slot * 8, parity);
        if (alive) {
            if (nsf > 0) la = l_addr();
#pragma unroll 1
            for (int t = 0; t < tail; ++t) {
                const uint32_t hw = lds16(fa + (uint32_t)t * D + pairA * 2) | (lds16(fa + (uint32_t)t * D + pairB * 2) << 16);
                const uint32_t lw = la ? lds16(la + (uint32_t)t * D + pairA * 2) | (lds16(la + (uint32_t)t * D + pairB * 2) << 16)
                                       : 0x80808080u;
                const uint32_t sb = lds16(sa + t * 2);
                accA = hfma2_bits(__byte_perm(hw, lw, 0x1504), sb | (sb << 16), accA);
                accB = hfma2_bits(__byte_perm(hw, lw, 0x3726), sb | (sb << 16), accB);
            }
        }
    }
    if (p.res) {
        const uint32_t* r = reinterpret_cast<const uint32_t*>(p.res) + (size_t)bh * 64;
        auto add = [](uint32_t acc, uint32_t t) {
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&acc));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t));
            const __half2 c = __floats2half2_rn(a.x + b.x, a.y + b.y);
            return *reinterpret_cast<const uint32_t*>(&c);
        };
        accA = add(accA, r[pairA]);
        accB = add(accB, r[pairB]);
    }
    uint32_t* o = reinterpret_cast<uint32_t*>(p.o) + (size_t)bh * 64;
    o[pairA] = alive ? accA : 0x7E007E00u;
    o[pairB] = alive ? accB : 0x7E007E00u;
}

}  // namespace akv
