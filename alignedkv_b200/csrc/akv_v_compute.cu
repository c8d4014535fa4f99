// Precision-aligned P.V over the quantized V tokens, and the magnitude probe that sets its threshold.
//
// Replaces the reference's v_cache_compute_kernel (extension/csrc/V_cache.cu:178-308) and
// v_cache_test_compute_kernel (V_cache.cu:90-123).  Outputs are bit-identical: each output channel is the fp16
// fused-multiply-add chain over tokens 0..n-1 in order, skipped nibble planes are replaced by the reference's
// constants (V_cache.cu:198-202,250-253).
//
// Design (B200): the exact token order leaves only B*Hq*D/2 independent chains - two warps per (batch, query head)
// - and a dependent fp16 FMA issues every ~4 cycles while every shared-memory load a warp issues costs it several
// more, so the kernel is organised around handing the chain warps operands they can take with few, wide loads.
// One CTA per (batch, KV head); the G query heads of a grouped-query group share the CTA and the bytes it streams.
//   producer warps (4: two pairs, pair p serves the 64-token stages j = p, p+2, ...; each warp of a pair serves one
//     run of 32 tokens of the stage).  (1) issue - thread = token: it takes each head's probability of the token from
//     a buffer bulk-copied 16 stages ahead, decides from its bit pattern which of the token's 64-byte nibble rows
//     are needed (V_cache.cu:211,250-251), and starts the copies: ONE bulk asynchronous copy (cp.async.bulk, the
//     TMA unit) for the stage's 8 KB of high bytes and 64-byte bulk copies of just the needed nibble rows into a
//     small side ring, all byte-counted on the stage's mbarrier; a few stages per pair are kept in flight.
//     (2) transform - once a stage has landed, the same warps transpose it into the "ready" ring as
//     [channel pair][token] 16-bit words (8x8 tiles, 16-byte accesses both ways, swizzled so that neither side has
//     bank conflicts) and - only for a run in which some token of a head reads a nibble plane - that head's
//     low-byte words, built from the side ring with the reference's substitutes (mid 0x88 / low 0x00 when neither
//     plane is read, low 0x88 when only mid is read).
//   chain warps (2 per query head; thread c owns channels 2c, 2c+1): per run of 32 tokens four 16-byte loads of
//     high words, eight of probability words, (four of low words when the run is not lean, else the constant 0x80
//     bytes), then per token one byte permute and one FMA.  The next run's loads and permutes are written between
//     the FMAs of the current one (software pipelining across runs and stages), so the chain sees ready operands.
//     A run has two code paths (lean / not lean), chosen once per run; there is no per-token branch.
// Every wait is time-bounded; a wait that gives up raises a flag the host can read (akv_device_error_flag).
#include "akv_v_chain.cuh"
#include "akv_v_stream.cuh"

namespace akv {

namespace vc {
constexpr int TOK = 64;   // tokens per stage
constexpr int RUN = 32;   // tokens per run (one loader warp's share of a stage)
constexpr int SCH = 16;   // stages per probability chunk
}

// Shared-memory plan of one CTA.
//   F ring      NF stages of 64 tokens x D high bytes as they lie in the plane, one bulk copy each
//   pending     per F slot: per run {side slot or -1, union mid mask, union low mask, -} and per query head
//               {mid mask, low mask} (bit u set = token u of the run reads that plane for that head), and per head
//               the 64 probability words (the fp16 value in both halves) the chain warps read
//   side ring   per producer warp NML slots of [32 tokens x D/2 mid bytes][32 tokens x D/2 low bytes]; only the rows
//               in the union masks are filled
//   ready ring  NR slots of: high words [64 pairs][64 tokens] (2 bytes each, 16-byte chunks swizzled) and per head
//               low words in the same layout (written only for runs that are not lean)
//   s chunks    three buffers of G x 16 stages x 64 probabilities.  Chunk c+1 is requested when the first producer
//               warp's issue side enters chunk c and lands in buffer (c+1) % 3, last read (by issue sides only)
//               during chunk c-2; the producer warps' issue positions are less than 16 stages apart.
//   barriers    landed per F slot, ready / free per ready slot, landed per probability buffer
// Stage j uses F slot j % NF and ready slot j % NR; NF and NR are even, so each producer pair owns every other slot.
template <int D, int G, int NF, int NR, int NML>
struct VPlan {
    static constexpr int TOK = vc::TOK;
    static constexpr int HD = D / 2;
    static constexpr int F_BYTES = TOK * D;
    static constexpr int PEND_OFF = NF * F_BYTES;
    static constexpr int REC_BYTES = (16 + G * 8 + 15) & ~15;                  // one run's record
    static constexpr int P_S2 = 2 * REC_BYTES;                                 // offsets inside a pending area
    static constexpr int PEND_BYTES = P_S2 + G * TOK * 4;
    static constexpr int ML_OFF = (PEND_OFF + NF * PEND_BYTES + 127) & ~127;
    static constexpr int ML_BYTES = vc::RUN * HD * 2;
    static constexpr int RDY_OFF = ML_OFF + 4 * NML * ML_BYTES;
    static constexpr int W_BYTES = HD * TOK * 2;                               // one [pair][token] array of 16-bit words
    static constexpr int R_LO = W_BYTES;                                       // offset inside a ready slot
    static constexpr int RDY_BYTES = (1 + G) * W_BYTES;
    static constexpr int SB_OFF = RDY_OFF + NR * RDY_BYTES;
    static constexpr int SB_HEAD = vc::SCH * TOK * 2;                          // bytes of one head's chunk
    static constexpr int SB_BYTES = G * SB_HEAD;                               // one buffer
    static constexpr int BAR_OFF = SB_OFF + 3 * SB_BYTES;
    static constexpr int BYTES = BAR_OFF + (NF + 2 * NR + 3) * 8;
    // Stages of one pair in flight beyond the one it transforms.  The pair's stage j + 2*AHEADP lands in the F slot
    // of stage j - NR - 2.  A warp reaches iteration j only after the chain released stage j - 2 - NR (it waited
    // for that to reuse the ready slot for stage j - 2), which also means both warps of the pair had published it:
    // nobody reads that F slot, its records or its probability words any more.
    static constexpr int AHEADP = NF / 2 - NR / 2 - 1;
    static_assert(NF % 2 == 0 && NR % 2 == 0 && AHEADP >= 1 && NF + NR + 4 < vc::SCH, "ring sizes");
    static_assert(PEND_BYTES % 16 == 0 && RDY_OFF % 128 == 0 && W_BYTES % 128 == 0, "alignment");
};

// 16-byte chunk k (tokens 8k..8k+7) of pair c's row in a [pair][token] array: swizzled so that a quarter-warp of
// consecutive pairs reading one chunk, and a quarter-warp of pair groups writing one pair, each hit 8 bank groups.
__device__ __forceinline__ uint32_t v_chunk(int c, int k) {
    return (uint32_t)c * 128u + (uint32_t)(((k ^ (c >> 3) ^ c) & 7) << 4);
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// 8 tokens x 8 pairs tile: R[j] = four words of token j (word i = pairs 2i, 2i+1, two bytes each) -> for pair q the
// 16 bytes of its 8 tokens, stored at the pair's swizzled chunk.  dst = array base; c0 = first pair, k = chunk index.
__device__ __forceinline__ void v_store_transposed(const uint4 (&R)[8], uint32_t dst, int c0, int k) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const uint32_t sel = (q & 1) ? 0x7632u : 0x5410u;
        uint32_t o[4];
#pragma unroll
        for (int m = 0; m < 4; ++m)   // [pair q of token 2m, pair q of token 2m+1]
            o[m] = __byte_perm(u4w(R[2 * m], q >> 1), u4w(R[2 * m + 1], q >> 1), sel);
        sts128(dst + v_chunk(c0 + q, k), o[0], o[1], o[2], o[3]);
    }
}

// 16-byte shared load that is only issued when `on` is non-zero; otherwise v keeps its value.
__device__ __forceinline__ void lds128_if(uint4& v, uint32_t a, uint32_t on) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %5, 0;\n@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n}\n"
                 : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w) : "r"(a), "r"(on));
}

// Low words of the run being fetched.  While runs are lean (no token of the run reads a nibble plane for this head)
// the registers simply keep the constant 0x80 bytes; they are refilled only when a lean run follows one that was not.
struct VLow {
    uint4 L[4];
    uint32_t dirty;
    __device__ __forceinline__ void fill() {
#pragma unroll
        for (int i = 0; i < 4; ++i) L[i] = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
        dirty = 0;
    }
};

// One run of 32 tokens of the chain.  KC / SC: the current run's k~ words [lo_even, f_even, lo_odd, f_odd] and
// probability words.  KN / SN receive the next run's: its 16-byte loads are written between the first sixteen FMAs and
// the byte permutes that build k~ between the last sixteen, so that all of it issues in the FMAs' latency shadow and
// the next run starts with operands that are ready.  FETCH == false: last run, nothing to load.  not_lean == 0
// (warp-uniform): the loads of the next run's low words are not issued and its low bytes are the constant 0x80 -
// one code path either way, which keeps the loop small enough for the instruction cache next to the producers' code.
template <bool FETCH>
__device__ __forceinline__ void v_run(uint32_t& acc, const uint32_t (&KC)[32], const uint4 (&SC)[8], uint32_t (&KN)[32],
                                      uint4 (&SN)[8], VLow& low, uint32_t hi_a, uint32_t lo_a, uint32_t s_a, int c,
                                      int k0, uint32_t not_lean) {
    uint4 H[4];
    // v_chunk(c, k) = v_chunk(c, 0) ^ (k << 4): the arrays are 128-byte aligned, so one XOR per load addresses a chunk
    const uint32_t hx = hi_a + v_chunk(c, 0), lx = lo_a + v_chunk(c, 0);
    if (FETCH) {
        if (not_lean == 0 && low.dirty) low.fill();   // (warp-uniform, rare)
        low.dirty |= not_lean;
    }
#pragma unroll
    for (int v = 0; v < 8; ++v) {          // 4 tokens per step
        if (FETCH) {
            SN[v] = lds128(s_a + v * 16);
            if (v < 4) {
                H[v] = lds128(hx ^ (uint32_t)((k0 + v) << 4));
                lds128_if(low.L[v], lx ^ (uint32_t)((k0 + v) << 4), not_lean);
            } else {
                const int i = v - 4;       // chunk i: word m holds tokens 8i+2m, 8i+2m+1
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    KN[8 * i + 2 * m] = __byte_perm(u4w(H[i], m), u4w(low.L[i], m), 0x1504);
                    KN[8 * i + 2 * m + 1] = __byte_perm(u4w(H[i], m), u4w(low.L[i], m), 0x3726);
                }
            }
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) acc = hfma2_bits(KC[4 * v + w], u4w(SC[v], w), acc);
    }
}

template <int D, int G, int NF, int NR, int NML>
__global__ void __launch_bounds__(64 * G + 128) v_compute_kernel(const VParams p) {
    using P = VPlan<D, G, NF, NR, NML>;
    constexpr int TOK = P::TOK;
    constexpr int NCH = 64 * G;                    // chain threads
    constexpr int HD = P::HD;                      // nibble row bytes
    static_assert(D == 128, "thread c of a head's two chain warps owns channels 2c, 2c+1");
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const long long bh = blockIdx.x;               // (batch, KV head)
    const int n = p.n;
    const int nst = (n + TOK - 1) / TOK;
    const uint32_t base = smem_u32(smem);
    const uint32_t bar_full = base + P::BAR_OFF, bar_ready = bar_full + NF * 8, bar_free = bar_ready + NR * 8;
    const uint32_t bar_sb = bar_free + NR * 8;

    pdl_enter();
    if (tid == 0) {
        for (int s = 0; s < NF; ++s) mbar_init(bar_full + s * 8, 2);   // one arrival per warp of the pair (+ bytes)
        for (int s = 0; s < NR; ++s) {
            mbar_init(bar_ready + s * 8, 2);         // one arrival per warp of the pair
            mbar_init(bar_free + s * 8, 2 * G);      // one arrival per chain warp
        }
        for (int s = 0; s < 3; ++s) mbar_init(bar_sb + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    if (tid < NCH) {
        // ------------------------------------------------------------------ chain warps
        const int g = tid >> 6, c = tid & 63, lane = tid & 31;
        const int nsf = n / TOK, tail = n - nsf * TOK;     // full stages, tokens of the partial last stage
        uint32_t acc = 0;
        uint32_t kA[32], kB[32];
        uint4 sA[8], sB[8];
        VLow low;
        low.fill();
#pragma unroll
        for (int u = 0; u < 32; ++u) kA[u] = kB[u] = 0;
#pragma unroll
        for (int v = 0; v < 8; ++v) sA[v] = sB[v] = make_uint4(0, 0, 0, 0);
        int rs = 0, fs = 0;        // ready slot and F slot of the stage whose first run is in the A registers
        uint32_t phase = 0;
        bool alive = true;
        auto rdy = [&](int r) { return base + P::RDY_OFF + (uint32_t)r * P::RDY_BYTES; };
        auto pend = [&](int f) { return base + P::PEND_OFF + (uint32_t)f * P::PEND_BYTES; };
        // "not lean" flag (this head's mid mask) of run `half` of the stage in F slot f
        auto flag = [&](int f, int half) { return lds32(pend(f) + half * P::REC_BYTES + 16 + g * 8); };
        uint32_t fl1 = 0;          // "not lean" flag of the second run of the stage in the A registers
        if (nsf > 0) {
            alive = mbar_wait(bar_ready, 0);
            if (alive) {   // (a chain over zeros) fetch run 0 of stage 0
                fl1 = flag(0, 1);
                v_run<true>(acc, kB, sB, kA, sA, low, rdy(0), rdy(0) + P::R_LO + g * P::W_BYTES,
                            pend(0) + P::P_S2 + g * TOK * 4, c, 0, flag(0, 0));
            }
        }
        for (int j = 0; j < nsf && alive; ++j) {
            const int nrs = rs + 1 == NR ? 0 : rs + 1, nfs = fs + 1 == NF ? 0 : fs + 1;
            const uint32_t nphase = rs + 1 == NR ? phase ^ 1 : phase;
            // first run of stage j while its second run is fetched
            v_run<true>(acc, kA, sA, kB, sB, low, rdy(rs), rdy(rs) + P::R_LO + g * P::W_BYTES,
                        pend(fs) + P::P_S2 + (g * TOK + vc::RUN) * 4, c, 4, fl1);
            // both runs of the stage are in registers: hand the ready slot (and with it the F slot's records and
            // probability words) back
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_free + rs * 8);
            // second run of stage j while the first run of stage j+1 is fetched.  The wait for stage j+1 comes as
            // late as this: between handing back a slot and needing its next content lie two runs, which is about
            // the time the producer pair needs to wake up and transform a stage (one run was not enough).
            if (j + 1 < nsf) {
                alive = mbar_wait(bar_ready + nrs * 8, nphase);
                if (!alive) break;
                fl1 = flag(nfs, 1);
                v_run<true>(acc, kB, sB, kA, sA, low, rdy(nrs), rdy(nrs) + P::R_LO + g * P::W_BYTES,
                            pend(nfs) + P::P_S2 + g * TOK * 4, c, 0, flag(nfs, 0));
            } else
                v_run<false>(acc, kB, sB, kA, sA, low, 0, 0, 0, c, 0, 0);
            rs = nrs; fs = nfs; phase = nphase;
        }
        if (tail > 0 && alive) {
            // last, partial stage: token by token from the ready slot
            alive = mbar_wait(bar_ready + rs * 8, phase);
            if (alive) {
                const uint32_t r = rdy(rs);
                const uint32_t f0 = flag(fs, 0), f1 = flag(fs, 1);
                for (int t = 0; t < tail; ++t) {
                    const uint32_t off = v_chunk(c, t >> 3) + (t & 7) * 2;
                    const uint32_t hw = lds16(r + off);
                    const uint32_t lw = ((t < vc::RUN) ? f0 : f1) ? lds16(r + P::R_LO + g * P::W_BYTES + off) : 0x8080u;
                    acc = hfma2_bits(__byte_perm(hw, lw, 0x1504), lds32(pend(fs) + P::P_S2 + (g * TOK + t) * 4), acc);
                }
            }
        }
        if (alive) reinterpret_cast<uint32_t*>(p.o)[((size_t)bh * G + g) * 64 + c] = acc;
        return;
    }

    // ---------------------------------------------------------------------- producer warps
    const int pt = tid - NCH, lane = pt & 31, pw = pt >> 5, pair = pw >> 1, half = pw & 1;
    const int tok = half * vc::RUN + lane;         // this thread's token of every stage of its pair
    const uint8_t* F = p.first8 + (size_t)bh * p.max_seq_len * D;
    const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * HD;
    const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * HD;
    const uint16_t* s_rows = p.s + (size_t)bh * G * p.s_last_dim;
    uint32_t A[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        uint32_t a;
        if (p.test_o) {
            a = v_threshold_warp(p.test_o, p.v_exp, bh * G + g, p.H, G, D, lane);
            if (pt == 0) p.amin_out[bh * G + g] = (uint8_t)a;
        } else {
            a = p.amin[bh * G + g];
        }
        A[g] = (a << 10) & 0xFFFFu;
    }
    // probability chunk c (stages 16c .. 16c+15 of every head) -> buffer c % 3; issued by one thread
    auto request_s = [&](int c) {
        const int t0 = c * vc::SCH * TOK;
        int cnt = n - t0;
        cnt = cnt > vc::SCH * TOK ? vc::SCH * TOK : cnt;
        const uint32_t bytes = (uint32_t)((cnt + 7) & ~7) * 2;     // rows are padded to a multiple of 8 values
        const uint32_t bar = bar_sb + (c % 3) * 8;
        mbar_arrive_expect(bar, bytes * G);
#pragma unroll
        for (int g = 0; g < G; ++g)
            bulk_copy(base + P::SB_OFF + (uint32_t)(c % 3) * P::SB_BYTES + g * P::SB_HEAD,
                      s_rows + (size_t)g * p.s_last_dim + t0, bytes, bar);
    };
    bool alive = true;
    int iss = pair;                     // next stage of this pair to issue
    int ml_alloc = 0, ml_freed = 0;     // side-ring slots this warp has handed out / taken back
    int last_chunk = -1;                // probability chunk the issue side has entered
    if (pt == 0 && nst > 0) request_s(0);

    // ---- issue: decisions and copies of stage i (this warp's run of it); false when it has to wait for a side slot
    auto issue = [&](int i) -> bool {
        const int fs = i % NF;
        const int t0 = i * TOK;
        const int cnt = (n - t0) < TOK ? (n - t0) : TOK;
        const int c = i / vc::SCH;
        if (c > last_chunk) {   // entering chunk c (once, even if this stage is retried): ask for the next one, make
            last_chunk = c;     // sure this one has landed
            if (pt == 0 && (c + 1) * vc::SCH < nst) request_s(c + 1);
            alive = alive && mbar_wait(bar_sb + (c % 3) * 8, (uint32_t)(c / 3) & 1u);
            if (!alive) return true;
        }
        // decisions from the bit patterns (V_cache.cu:211,250-251): 16-bit wrap-around, signed compare
        const uint32_t sbase = base + P::SB_OFF + (uint32_t)(c % 3) * P::SB_BYTES + (i - c * vc::SCH) * (TOK * 2) + tok * 2;
        uint32_t mm[G], lm[G], sb[G];
        int ucode = 2;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            // (beyond the last token the buffer holds stale but readable bytes; the code below ignores them)
            sb[g] = lds16(sbase + g * P::SB_HEAD);
            if (tok >= cnt) sb[g] = 0u;
            const int diff = (int)(int16_t)(uint16_t)(A[g] - sb[g]);
            int code = p.reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
            if (tok >= cnt) code = 2;
            mm[g] = __ballot_sync(0xFFFFFFFFu, code < 2);
            lm[g] = __ballot_sync(0xFFFFFFFFu, code == 0);
            ucode = code < ucode ? code : ucode;
        }
        // union over the heads of the group (with one head it is that head's masks)
        const uint32_t umm = G == 1 ? mm[0] : __ballot_sync(0xFFFFFFFFu, ucode < 2);
        const uint32_t ulm = G == 1 ? lm[0] : __ballot_sync(0xFFFFFFFFu, ucode == 0);
        int ms = -1;
        uint32_t bytes = (half == 0) ? (uint32_t)cnt * D : 0u;
        if (umm) {
            // the rows some head reads go to a slot of this warp's side ring (freed by this warp's own transform)
            if (ml_alloc - ml_freed == NML) return false;
            ms = ml_alloc % NML;
            ++ml_alloc;
            bytes += (uint32_t)HD * (__popc(umm) + __popc(ulm));
        }
        const uint32_t bar = bar_full + fs * 8;
        const uint32_t pa = base + P::PEND_OFF + (uint32_t)fs * P::PEND_BYTES;
#pragma unroll
        for (int g = 0; g < G; ++g)
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(pa + P::P_S2 + (g * TOK + tok) * 4), "r"(sb[g] | (sb[g] << 16)) : "memory");
        if (lane == 0) {
            const uint32_t ra = pa + half * P::REC_BYTES;
            sts128(ra, (uint32_t)ms, umm, ulm, 0u);
#pragma unroll
            for (int g = 0; g < G; ++g)
                asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(ra + 16 + g * 8), "r"(mm[g]), "r"(lm[g]) : "memory");
        }
        __syncwarp();
        if (lane == 0) {
            if (bytes) mbar_arrive_expect(bar, bytes);   // publishes this warp's stores, announces its copies
            else mbar_arrive(bar);
        }
        if (half == 0 && lane == 0) bulk_copy(base + (uint32_t)fs * P::F_BYTES, F + (size_t)t0 * D, (uint32_t)cnt * D, bar);
        if (umm) {
            const uint32_t dm = base + P::ML_OFF + (uint32_t)(pw * NML + ms) * P::ML_BYTES;
            const size_t src = (size_t)(t0 + half * vc::RUN) * HD;
            // a run that reads a plane for all 32 tokens takes it as one 2 KB copy, otherwise row by row
            if (umm == 0xFFFFFFFFu) { if (lane == 0) bulk_copy(dm, M + src, vc::RUN * HD, bar); }
            else if (ucode < 2) bulk_copy(dm + lane * HD, M + src + (size_t)lane * HD, HD, bar);
            if (ulm == 0xFFFFFFFFu) { if (lane == 0) bulk_copy(dm + vc::RUN * HD, L + src, vc::RUN * HD, bar); }
            else if (ucode == 0) bulk_copy(dm + (vc::RUN + lane) * HD, L + src + (size_t)lane * HD, HD, bar);
        }
        return true;
    };

    const int tg = 4 * half + (lane >> 3), pg = lane & 7;      // this lane's 8-token x 8-pair tile of every stage
    for (int j = pair; j < nst && alive; j += 2) {
        // keep AHEADP stages of this pair in flight beyond the one transformed now
        while (alive && iss < nst && iss <= j + 2 * P::AHEADP) {
            if (!issue(iss)) break;
            iss += 2;
        }
        if (!alive) break;
        const int fs = j % NF, rs = j % NR;
        alive = mbar_wait(bar_full + fs * 8, (uint32_t)(j / NF) & 1u);                       // the stage has landed
        if (alive && j >= NR) alive = mbar_wait(bar_free + rs * 8, (uint32_t)(j / NR - 1) & 1u);   // slot consumed
        if (!alive) break;
        const uint32_t fa = base + (uint32_t)fs * P::F_BYTES, r = base + P::RDY_OFF + (uint32_t)rs * P::RDY_BYTES;
        const uint32_t ra = base + P::PEND_OFF + (uint32_t)fs * P::PEND_BYTES + half * P::REC_BYTES;
        // high bytes: transpose this lane's tile
        {
            uint4 R[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) R[t] = lds128(fa + (8 * tg + t) * D + pg * 16);
            v_store_transposed(R, r, 8 * pg, tg);
        }
        // low bytes, only for the heads that read a nibble plane in this warp's run
        const uint32_t umm = lds32(ra + 4);
        if (umm) {
            const int ms = (int)lds32(ra);
            const uint32_t mla = base + P::ML_OFF + (uint32_t)(pw * NML + ms) * P::ML_BYTES;
            const int u0 = 8 * (lane >> 3);                       // first token of the tile inside the run
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const uint2 hm = lds64(ra + 16 + g * 8);
                if (hm.x == 0) continue;                          // (warp-uniform)
                uint4 R[8];
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    uint2 mb = lds64(mla + (u0 + t) * HD + pg * 8);
                    uint2 lb = lds64(mla + (vc::RUN + u0 + t) * HD + pg * 8);
                    const bool m = (hm.x >> (u0 + t)) & 1u, l = (hm.y >> (u0 + t)) & 1u;
                    if (!m) mb = make_uint2(0x88888888u, 0x88888888u);
                    if (!l) lb = m ? make_uint2(0x88888888u, 0x88888888u) : make_uint2(0u, 0u);
                    const uint32_t le0 = (mb.x & 0xF0F0F0F0u) | ((lb.x >> 4) & 0x0F0F0F0Fu);   // even channels, pairs 0-3
                    const uint32_t le1 = (mb.y & 0xF0F0F0F0u) | ((lb.y >> 4) & 0x0F0F0F0Fu);   //                pairs 4-7
                    const uint32_t lo0 = ((mb.x << 4) & 0xF0F0F0F0u) | (lb.x & 0x0F0F0F0Fu);   // odd channels
                    const uint32_t lo1 = ((mb.y << 4) & 0xF0F0F0F0u) | (lb.y & 0x0F0F0F0Fu);
                    R[t].x = __byte_perm(le0, lo0, 0x5140);       // pairs 0,1: [even, odd, even, odd]
                    R[t].y = __byte_perm(le0, lo0, 0x7362);       // pairs 2,3
                    R[t].z = __byte_perm(le1, lo1, 0x5140);
                    R[t].w = __byte_perm(le1, lo1, 0x7362);
                }
                v_store_transposed(R, r + P::R_LO + g * P::W_BYTES, 8 * pg, tg);
            }
            ++ml_freed;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ready + rs * 8);
    }
    if (!alive) {
        // a wait gave up (never expected): give the copies already in flight time to land before the CTA's shared
        // memory is released
        for (int i = 0; i < 2000; ++i) __nanosleep(100);
    }
}

// Any even head_dim, any group size: one thread per channel pair, planes read straight from global memory.
__global__ void __launch_bounds__(128)
v_compute_generic_kernel(const VParams p, int bhq_count) {
    const int hd = p.D >> 1;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)bhq_count * hd;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % hd);
        const long long bhq = i / hd, bh = bhq / p.group;
        const uint8_t* F = p.first8 + (size_t)bh * p.max_seq_len * p.D;
        const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * hd;
        const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * hd;
        const uint16_t* s_row = p.s + (size_t)bhq * p.s_last_dim;
        const uint32_t A = ((uint32_t)p.amin[bhq] << 10) & 0xFFFFu;
        uint32_t acc = 0;
        for (int t = 0; t < p.n; ++t) {
            const uint32_t sb = s_row[t];
            const int diff = (int)(int16_t)(uint16_t)(A - sb);
            const int code = p.reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
            const uint32_t f = *reinterpret_cast<const uint16_t*>(F + (size_t)t * p.D + 2 * c);
            uint32_t mb = 0x88u, lb = 0x00u;
            if (code < 2) {
                mb = M[(size_t)t * hd + c];
                lb = (code == 0) ? (uint32_t)L[(size_t)t * hd + c] : 0x88u;
            }
            const uint32_t lo = ((mb & 0xF0u) | (lb >> 4)) | ((((mb & 0x0Fu) << 4) | (lb & 0x0Fu)) << 8);
            acc = hfma2_bits(__byte_perm(f, lo, 0x1504), sb | (sb << 16), acc);
        }
        reinterpret_cast<uint32_t*>(p.o)[(size_t)bhq * hd + c] = acc;
    }
}

template <int G, int NF, int NR, int NML>
static int launch_v_fast(const VParams& p, int BH, cudaStream_t st) {
    using K = VPlan<128, G, NF, NR, NML>;
    static bool configured[64] = {false};   // the attribute is per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(v_compute_kernel<128, G, NF, NR, NML>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)K::BYTES);
        if (e != cudaSuccess) return cuda_status(e, "v_cache_compute smem attribute");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    launch_chained(v_compute_kernel<128, G, NF, NR, NML>, dim3(BH), dim3(64 * G + 128), K::BYTES, st, p);
    return cuda_status(cudaGetLastError(), "v_cache_compute launch");
}

// ---- launch of the branch-free streaming form for multi-head attention (v_chain_kernel)
// Ring sizes follow from how many units ((batch, head) pairs) have to share an SM so that the whole grid is resident
// at once (the kernel is a pure stream: a second wave would start with cold rings): shared memory per unit = SM
// capacity / units per SM, of which the probability buffers and the side ring take a fixed part and the two rings
// (high bytes, low-byte table: 16 KB per stage) the rest.
struct VChainCfg {
    int upc, gh, ndw, nf, nside, sch, npt, smem;
};
// heads: (batch, query head) rows; gh: heads that share a ring (1, or the group size: the query heads of a KV head)
static VChainCfg v_chain_config(long long heads, int gh, int reference) {
    const Tuning& t = tuning();
    VChainCfg c;
    c.gh = gh;
    // one head per ring: two rings per CTA, whose eight warps put the chain and decision warps on different schedulers
    c.upc = (gh == 1 && heads >= 2) ? 2 : 1;
    if (gh == 1 && t.v_upc > 0) c.upc = t.v_upc;
    const int budget = max_dyn_smem();
    // decision warps per head: a stage with flagged tokens costs its warp three out-of-line calls (copy issue, row
    // build, row restore), and two warps per head fell behind the chain on them; four have the time.  They need
    // schedulers of their own, which two rings of one head each can give them.
    c.ndw = (c.upc == 2 && gh == 1 && tuning().v_ndw != 2) ? 4 : 2;
    c.nside = (reference ? 128 : 64) * c.ndw;              // (each decision warp owns a part: at least a stage's 64 rows)
    c.sch = 16;
    if (t.v_nside >= 64 * c.ndw) c.nside = t.v_nside;
    // low-byte tables per head: two per decision warp where they fit (a third stage with flagged tokens among a warp's
    // stages in flight is rare and only makes that warp wait for the oldest one), one with four heads on a ring
    c.npt = c.upc * gh >= 4 ? 2 : 4;
    if (t.v_npt == 2 || t.v_npt == 4 || t.v_npt == 6 || t.v_npt == 8) c.npt = t.v_npt;
    // ring depth: the decision warp runs a ring ahead, 2 nf stages <= a chunk; one head per ring gains nothing beyond
    // four stages (measured: 4, 6 and 8 alike), heads that share a ring wait for each other and use what fits
    int nf = gh == 1 ? 4 : c.sch / 2;
    if (t.v_nf > 0 && t.v_nf < nf) nf = t.v_nf;
    nf -= nf % c.ndw;                                      // a ring slot's stages all belong to one decision warp
    if (nf < c.ndw) nf = c.ndw;
    // (one head per ring: a table per ring slot)
    while (nf > c.ndw && vch::plan(nf, c.nside, c.sch, gh == 1 ? nf : c.npt, c.upc, gh).bytes > budget) nf -= c.ndw;
    c.nf = nf;
    if (gh == 1) c.npt = nf;
    c.smem = vch::plan(c.nf, c.nside, c.sch, c.npt, c.upc, gh).bytes;
    return c;
}

template <int UPC, int GH, int NDW>
static int launch_v_chain_u(VParams& p, const VChainCfg& c, long long heads, cudaStream_t st) {
    static bool configured[64] = {false};   // the attribute is per device (one array per instantiation)
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(v_chain_kernel<UPC, GH, NDW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             max_dyn_smem());
        if (e != cudaSuccess) return cuda_status(e, "v_cache_compute smem attribute");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    AKV_REQUIRE(c.smem <= max_dyn_smem(), AKV_ERR_CUDA, "v_cache_compute: %d bytes of shared memory are too many", c.smem);
    p.nf = c.nf; p.nside = c.nside; p.sch = c.sch; p.npt = c.npt;
    p.units = (int)(heads / GH);
    const int grid = (p.units + UPC - 1) / UPC;
    launch_chained(v_chain_kernel<UPC, GH, NDW>, dim3(grid), dim3(NDW == 2 ? ((1 + NDW) * UPC * GH + UPC) * 32 : 512), (size_t)c.smem, st, p);
    return cuda_status(cudaGetLastError(), "v_cache_compute launch");
}

// true when launch_v_compute_probe runs the streaming kernel, which can compute the threshold bytes itself
bool v_compute_takes_probe(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                           const uint8_t* o, int group, int D, int s_last_dim, int n) {
    return D == 128 && (group == 1 || group == 2 || group == 4) &&
           aligned16(first8) && aligned16(mid4) &&
           aligned16(last4) && (n == 0 || (aligned16(s) && s_last_dim % 8 == 0 && ((n + 7) & ~7) <= s_last_dim)) &&
           ((reinterpret_cast<uintptr_t>(o) & 3u) == 0);
}

// P.V over n quantized tokens.  H = KV heads, group = query heads per KV head; s rows, amin bytes and output rows
// are per (batch, query head) with query head = KV head * group + g.  test_o != nullptr (only when
// v_compute_takes_probe() holds): the threshold bytes are computed in the kernel from the probe result and the
// exponent maxima v_exp and written to amin_out; otherwise they are read from amin.
// res != nullptr (only when v_compute_adds_residual() holds): the kernel adds res [B, Hq, D] (fp16) to its result.
int launch_v_compute_res(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                         uint8_t* amin, const uint8_t* test_o, const uint8_t* v_exp, const uint8_t* res, uint8_t* o,
                         int bsz, int H, int group, int max_seq_len, int D, int s_last_dim, int n, int reference,
                         cudaStream_t st) {
    VParams p;
    p.res = reinterpret_cast<const uint16_t*>(res);
    p.first8 = first8; p.mid4 = mid4; p.last4 = last4;
    p.s = reinterpret_cast<const uint16_t*>(s);
    p.amin = amin;
    p.test_o = reinterpret_cast<const uint16_t*>(test_o); p.v_exp = v_exp; p.amin_out = amin; p.H = H;
    p.o = reinterpret_cast<uint16_t*>(o);
    p.max_seq_len = max_seq_len; p.D = D; p.s_last_dim = s_last_dim; p.n = n; p.reference = reference;
    p.group = group;
    p.nf = p.nside = p.sch = p.units = 0;
    const int BH = bsz * H;
    const bool fast = v_compute_takes_probe(first8, mid4, last4, s, o, group, D, s_last_dim, n);
    AKV_REQUIRE(fast || !test_o, AKV_ERR_SHAPE, "v_cache_compute: the probe form needs the streaming kernel");
    const long long heads = (long long)BH * group;
    const bool chain = fast && !reference && tuning().v_impl == 0 && heads < (1ll << 30);
    AKV_REQUIRE(chain || !p.res, AKV_ERR_SHAPE, "v_cache_compute: the residual form needs the chain kernel");
    if (chain) {
        // grouped queries: the heads of a KV head share one ring of high bytes in a CTA (gh = group); the form with
        // one ring per query head, whose heads meet in L2, stays selectable for measurements
        // (measured at 8192 tokens, 8 KV heads x 4: batch 8: 98 us grouped kernel, 84 shared ring, 65 ring per head;
        // batch 16: 117 / 102 / 125): a ring per head while the heads fit one wave of CTAs, else the shared ring
        const int w = tuning().v_gqa_form;
        const bool per_head = group == 1 || w == 1 || (w == 0 && heads <= 2ll * sm_count());
        const int gh = per_head ? 1 : group;
        const VChainCfg c = v_chain_config(heads, gh, reference);
        if (gh == 4) return launch_v_chain_u<1, 4, 2>(p, c, heads, st);
        if (gh == 2) return launch_v_chain_u<1, 2, 2>(p, c, heads, st);
        if (c.upc == 2) return c.ndw == 4 ? launch_v_chain_u<2, 1, 4>(p, c, heads, st) : launch_v_chain_u<2, 1, 2>(p, c, heads, st);
        return launch_v_chain_u<1, 1, 2>(p, c, heads, st);
    }
    if (fast && group == 1) return launch_v_fast<1, 6, 2, 1>(p, BH, st);
    if (fast && group == 2) return launch_v_fast<2, 6, 2, 2>(p, BH, st);
    if (fast && group == 4) return launch_v_fast<4, 6, 2, 2>(p, BH, st);
    long long total = (long long)BH * group * (D >> 1);
    long long want = (total + 127) / 128;
    int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
    if (grid < 1) grid = 1;
    count_launch();
    v_compute_generic_kernel<<<grid, 128, 0, st>>>(p, BH * group);
    return cuda_status(cudaGetLastError(), "v_cache_compute launch");
}

int launch_v_compute_probe(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                           uint8_t* amin, const uint8_t* test_o, const uint8_t* v_exp, uint8_t* o, int bsz, int H,
                           int group, int max_seq_len, int D, int s_last_dim, int n, int reference, cudaStream_t st) {
    return launch_v_compute_res(first8, mid4, last4, s, amin, test_o, v_exp, nullptr, o, bsz, H, group, max_seq_len, D,
                                s_last_dim, n, reference, st);
}

// true when launch_v_compute_res runs the chain kernel, which can add the residual tokens' part to its result
bool v_compute_adds_residual(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                             const uint8_t* o, int bsz, int H, int group, int D, int s_last_dim, int n, int reference) {
    return v_compute_takes_probe(first8, mid4, last4, s, o, group, D, s_last_dim, n) && !reference &&
           tuning().v_impl == 0 && (long long)bsz * H * group < (1ll << 30);
}

int launch_v_compute(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                     const uint8_t* amin, uint8_t* o, int bsz, int H, int group, int max_seq_len, int D,
                     int s_last_dim, int n, int reference, cudaStream_t st) {
    return launch_v_compute_probe(first8, mid4, last4, s, const_cast<uint8_t*>(amin), nullptr, nullptr, o, bsz, H, group,
                                  max_seq_len, D, s_last_dim, n, reference, st);
}

// ================================================================== probe
// o_test[b,h,d] = sum_j |half((first_8[row_j][d] << 8) + 0x80)| * s_val[j], rows row_j = idx_j * K + j,
// accumulated in fp16 in j order (V_cache.cu:104-119).  All K row gathers are issued before the chain starts.
template <int KMAX>
__global__ void __launch_bounds__(128)
v_probe_kernel(const uint8_t* __restrict__ first8, const uint16_t* __restrict__ s_val,
               const int32_t* __restrict__ s_idx, uint16_t* __restrict__ out, int max_seq_len, int D, int K, int G) {
    pdl_enter();
    const long long bh = blockIdx.x;                                    // (batch, query head)
    const uint8_t* F = first8 + (size_t)(bh / G) * max_seq_len * D;     // planes of its KV head
    for (int c = threadIdx.x; c < (D >> 1); c += blockDim.x) {
        uint32_t acc = 0;
        for (int j0 = 0; j0 < K; j0 += KMAX) {
            uint32_t f[KMAX], sv[KMAX];
#pragma unroll
            for (int u = 0; u < KMAX; ++u) {
                const int j = j0 + u;
                f[u] = 0;
                sv[u] = 0;
                if (j < K) {
                    long long row = (long long)__ldg(s_idx + bh * K + j) * K + j;
                    row = row < 0 ? 0 : (row >= max_seq_len ? max_seq_len - 1 : row);
                    f[u] = __ldg(reinterpret_cast<const uint16_t*>(F + (size_t)row * D + 2 * c));
                    sv[u] = __ldg(s_val + bh * K + j);
                }
            }
#pragma unroll
            for (int u = 0; u < KMAX; ++u) {
                if (j0 + u < K) {
                    const uint32_t v = __byte_perm(f[u], 0x80u, 0x1404) & 0x7FFF7FFFu;  // |(f<<8) + 0x80| per half
                    acc = hfma2_bits(v, sv[u] | (sv[u] << 16), acc);
                }
            }
        }
        reinterpret_cast<uint32_t*>(out)[(size_t)bh * (D >> 1) + c] = acc;
    }
}

int launch_v_probe(const uint8_t* first8, const uint8_t* s_val, const uint8_t* s_idx, uint8_t* out, int bsz, int H,
                   int group, int max_seq_len, int D, int K, cudaStream_t st) {
    int threads = (D >> 1) < 128 ? (((D >> 1) + 31) / 32) * 32 : 128;
    launch_chained(v_probe_kernel<32>, dim3(bsz * H * group), dim3(threads), 0, st, first8,
                   reinterpret_cast<const uint16_t*>(s_val), reinterpret_cast<const int32_t*>(s_idx),
                   reinterpret_cast<uint16_t*>(out), max_seq_len, D, K, group);
    return cuda_status(cudaGetLastError(), "v_cache_test_compute launch");
}

// Split pass of the order-free P.V in its streaming form (akv_v_stream.cuh), for akv_v_split.cu.
int launch_v_split_stream(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                          uint8_t* amin, const uint8_t* test_o, const uint8_t* v_exp, int H, float* partial, int BH,
                          int max_seq_len, int s_last_dim, int n, int chunk_tokens, int chunks, cudaStream_t st) {
    VStreamParams p;
    p.first8 = first8; p.mid4 = mid4; p.last4 = last4;
    p.s = reinterpret_cast<const uint16_t*>(s);
    p.amin = amin; p.partial = partial;
    p.test_o = reinterpret_cast<const uint16_t*>(test_o); p.v_exp = v_exp; p.amin_out = amin; p.H = H;
    p.max_seq_len = max_seq_len; p.s_last_dim = s_last_dim; p.n = n;
    p.chunk_tokens = chunk_tokens; p.chunks = chunks; p.nf = 0;
    return launch_v_stream(p, BH, st);
}

// (the peer exchange kernel keeps a flag of its own: akv_exchange.cu)
unsigned int exchange_error_flag(cudaError_t* e);
cudaError_t exchange_error_clear();

}  // namespace akv

extern "C" int akv_device_error_flag(void) {
    // Non-zero once a bounded wait inside a kernel of this library gave up (never expected; the kernel then
    // returned early and its output is invalid).  Reading the flag synchronises the device.
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, akv::g_v_wait_gave_up, sizeof(v));
    if (e != cudaSuccess) return akv::cuda_status(e, "device_error_flag");
    v |= akv::exchange_error_flag(&e);
    if (e != cudaSuccess) return akv::cuda_status(e, "device_error_flag");
    return (int)v;
}

extern "C" int akv_device_error_clear(void) {
    // Puts the flag back to zero (after the caller has dealt with a run that raised it).  Synchronises the device.
    const unsigned int v = 0;
    cudaError_t e = cudaMemcpyToSymbol(akv::g_v_wait_gave_up, &v, sizeof(v));
    if (e == cudaSuccess) e = akv::exchange_error_clear();
    if (e != cudaSuccess) return akv::cuda_status(e, "device_error_clear");
    return AKV_OK;
}
