// Precision-aligned P.V over the quantized V tokens, and the magnitude probe that sets its threshold.
//
// Replaces the reference's v_cache_compute_kernel (extension/csrc/V_cache.cu:178-308) and
// v_cache_test_compute_kernel (V_cache.cu:90-123).  Outputs are bit-identical: each output channel is the fp16
// fused-multiply-add chain over tokens 0..n-1 in order, skipped nibble planes are replaced by the reference's
// constants (V_cache.cu:198-202,250-253).
//
// Design (B200): the exact token order leaves only B*Hq*D/2 independent chains - two warps per (batch, query head)
// - and a dependent fp16 FMA issues every ~4 cycles, so the kernel is organised around keeping those warps'
// instruction stream at one FMA plus its operand fetch per token and never letting them wait for memory.
// One CTA per (batch, KV head); the G query heads of a grouped-query group share the CTA and the bytes it streams.
//   chain warps (2 per query head; thread c owns channels 2c, 2c+1): tokens are handled in runs of 32.  While the
//     32 dependent FMAs of one run execute, the operands of the next run are fetched from shared memory into
//     registers in the FMAs' shadow (software pipelining across runs and across stages).  A run in which no token
//     of this head reads a nibble plane ("lean") costs one 2-byte load and one byte permute per token.
//   loader warps (64 threads; thread t owns token t of every 64-token stage): take each head's probability of the
//     token from a buffer that is copied 16 stages ahead, decide from its bit pattern which of the token's 64-byte
//     nibble rows are needed (V_cache.cu:211,250-251), and start the copies: ONE bulk asynchronous copy
//     (cp.async.bulk, the TMA unit) for the stage's 8 KB of high bytes, and 64-byte bulk copies for just the
//     needed nibble rows into a small side ring.  All copies complete on the stage's mbarrier by byte count, so a
//     loader never waits for data, only for a free slot.
// Every wait is a bounded spin; a wait that gives up raises a flag the host can read (akv_device_error_flag).
#include "akv_common.cuh"

namespace akv {

namespace vc {
constexpr int TOK = 64;   // tokens per stage
constexpr int RUN = 32;   // tokens per run (one loader warp's share of a stage)
constexpr int SCH = 16;   // stages per probability chunk
}

struct VParams {
    const uint8_t* first8;
    const uint8_t* mid4;
    const uint8_t* last4;
    const uint16_t* s;      // probabilities, one row per (batch, query head)
    const uint8_t* amin;    // threshold byte per (batch, query head)
    uint16_t* o;            // [B, Hq, D]
    int max_seq_len, D, s_last_dim, n, reference;
    int group;              // query heads per KV head (1 = multi-head attention)
};


// ---- shared-memory barriers (mbarrier) with bounded waits
static __device__ unsigned int g_v_wait_gave_up = 0;

   // set when a bounded wait ran out (never expected)

__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(a) : "memory");
}
// arrives and adds `bytes` to the byte count the current phase still waits for
__device__ __forceinline__ void mbar_arrive_expect(uint32_t a, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(a), "r"(bytes) : "memory");
}
// Bounded wait: gives up (and raises the device error flag) after about 20 ms.
__device__ __forceinline__ bool mbar_wait(uint32_t a, uint32_t parity) {
    unsigned long long t0 = 0;
    for (int spin = 0; spin < (1 << 24); ++spin) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
        if ((spin & 63) == 63) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > 20000000ull) break;
        }
    }
    atomicOr(&g_v_wait_gave_up, 1u);
    return false;
}
// Bulk asynchronous copy global -> shared through the TMA unit; 16-byte aligned addresses, size a multiple of 16.
// Completion is signalled on the mbarrier as `bytes` of its pending byte count.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Shared-memory plan of one CTA.
//   F ring     NS stages of 64 tokens x D high bytes, one bulk copy each
//   s2 ring    per stage and query head: 64 probability words (the fp16 value in both halves)
//   records    per stage and run of 32 tokens: {side slot or -1, union mid mask, union low mask, -} and per query
//              head {mid mask, low mask}: bit u set = token u of the run reads that plane for that head
//   side ring  per loader warp NML slots of [32 tokens x D/2 mid bytes][32 tokens x D/2 low bytes]; only the rows
//              in the union masks are filled
//   s chunks   three buffers of G x 16 stages x 64 probabilities.  Chunk c+1 is requested by one thread when it
//              enters chunk c and lands in buffer (c+1) % 3, last read during chunk c-2; the other loader warp is
//              in chunk c-1 or later because the ring (NS <= 16 stages) is shorter than a chunk.
//   barriers   full / empty per stage, free per side-ring slot, landed per probability buffer
template <int D, int G, int NS, int NML>
struct VPlan {
    static constexpr int TOK = vc::TOK;
    static constexpr int HD = D / 2;
    static constexpr int F_BYTES = TOK * D;
    static constexpr int S2_OFF = NS * F_BYTES;
    static constexpr int S2_BYTES = G * TOK * 4;
    static constexpr int REC_OFF = S2_OFF + NS * S2_BYTES;
    static constexpr int REC_BYTES = (16 + G * 8 + 15) & ~15;
    static constexpr int ML_OFF = (REC_OFF + NS * 2 * REC_BYTES + 127) & ~127;
    static constexpr int ML_BYTES = vc::RUN * HD * 2;
    static constexpr int SB_OFF = ML_OFF + 2 * NML * ML_BYTES;
    static constexpr int SB_HEAD = vc::SCH * TOK * 2;          // bytes of one head's chunk
    static constexpr int SB_BYTES = G * SB_HEAD;               // one buffer
    static constexpr int BAR_OFF = SB_OFF + 3 * SB_BYTES;
    static constexpr int BYTES = BAR_OFF + (2 * NS + 2 * NML + 3) * 8;
};

// One run of 32 tokens of the chain, with the next run's operand fetch written between the dependent FMAs so that
// the loads issue in the FMAs' latency shadow (they run AKV_V_PD tokens ahead of the FMA they are written next to).
// KC / SC: operands of the current run (k~ words [lo_even, f_even, lo_odd, f_odd], probability words); KN / SN
// receive the next run's.
//   AKV_V_RUN_NONE  nothing to fetch (last run)
//   AKV_V_RUN_LEAN  the next run's low bytes are the constant 0x80 (no nibble plane read)
//   AKV_V_RUN_FULL  nibble bytes come from the side ring where the head's masks say so, else the reference's
//                   substitutes (mid 0x88 / low 0x00 when neither plane is read, low 0x88 when only mid is read)
//   AKV_V_PATCH     after a lean fetch: rebuild the few tokens whose mask bit is set (cheaper than a full fetch when
//                   only one or two tokens of the run read a nibble plane, the common case)
#define AKV_V_PD 8
#define AKV_V_S(S_, v_, w_) ((w_) == 0 ? S_[v_].x : (w_) == 1 ? S_[v_].y : (w_) == 2 ? S_[v_].z : S_[v_].w)
#define AKV_V_RUN_NONE(KC_, SC_)                                                         \
    _Pragma("unroll") for (int v_ = 0; v_ < 8; ++v_) {                                   \
        _Pragma("unroll") for (int w_ = 0; w_ < 4; ++w_)                                 \
            acc = hfma2_bits(KC_[4 * v_ + w_], AKV_V_S(SC_, v_, w_), acc);               \
    }
#define AKV_V_RUN_LEAN(KC_, SC_, KN_, SN_, fa_, sa_)                                     \
    {                                                                                    \
        uint32_t raw_[32];                                                               \
        _Pragma("unroll") for (int v_ = 0; v_ < 8; ++v_) SN_[v_] = lds128((sa_) + v_ * 16); \
        _Pragma("unroll") for (int u_ = 0; u_ < AKV_V_PD; ++u_) raw_[u_] = lds16((fa_) + u_ * D); \
        _Pragma("unroll") for (int v_ = 0; v_ < 8; ++v_) {                               \
            _Pragma("unroll") for (int w_ = 0; w_ < 4; ++w_) {                           \
                const int u_ = 4 * v_ + w_;                                              \
                if (u_ + AKV_V_PD < 32) raw_[u_ + AKV_V_PD] = lds16((fa_) + (u_ + AKV_V_PD) * D); \
                acc = hfma2_bits(KC_[u_], AKV_V_S(SC_, v_, w_), acc);                    \
                KN_[u_] = __byte_perm(raw_[u_], 0x80u, 0x1404);                          \
            }                                                                            \
        }                                                                                \
    }
#define AKV_V_ASSEMBLE(f_, mb_, lb_) \
    __byte_perm((f_), (((mb_) & 0xF0u) | ((lb_) >> 4)) | (((((mb_) << 4) & 0xF0u) | ((lb_) & 0x0Fu)) << 8), 0x1504)
#define AKV_V_RUN_FULL(KC_, SC_, KN_, SN_, fa_, sa_, mla_, mm_, lm_)                     \
    _Pragma("unroll") for (int v_ = 0; v_ < 8; ++v_) {                                   \
        SN_[v_] = lds128((sa_) + v_ * 16);                                               \
        _Pragma("unroll") for (int w_ = 0; w_ < 4; ++w_) {                               \
            const int u_ = 4 * v_ + w_;                                                  \
            acc = hfma2_bits(KC_[u_], AKV_V_S(SC_, v_, w_), acc);                        \
            const uint32_t f_ = lds16((fa_) + u_ * D);                                   \
            uint32_t mb_ = lds8((mla_) + u_ * HD), lb_ = lds8((mla_) + (32 + u_) * HD);  \
            const bool m_ = ((mm_) >> u_) & 1u, l_ = ((lm_) >> u_) & 1u;                 \
            mb_ = m_ ? mb_ : 0x88u;                                                      \
            lb_ = l_ ? lb_ : (m_ ? 0x88u : 0x00u);                                       \
            KN_[u_] = AKV_V_ASSEMBLE(f_, mb_, lb_);                                      \
        }                                                                                \
    }
#define AKV_V_PATCH(KN_, fa_, mla_, mm_, lm_)                                            \
    for (uint32_t rem_ = (mm_); rem_; rem_ &= rem_ - 1) {                                \
        const int t_ = __ffs((int)rem_) - 1;                                             \
        const uint32_t f_ = lds16((fa_) + t_ * D);                                       \
        const uint32_t mb_ = lds8((mla_) + t_ * HD);                                     \
        uint32_t lb_ = lds8((mla_) + (32 + t_) * HD);                                    \
        lb_ = (((lm_) >> t_) & 1u) ? lb_ : 0x88u;                                        \
        const uint32_t w_ = AKV_V_ASSEMBLE(f_, mb_, lb_);                                \
        _Pragma("unroll") for (int u_ = 0; u_ < 32; ++u_) KN_[u_] = (u_ == t_) ? w_ : KN_[u_]; \
    }
// Run over KC/SC while fetching run `half_` of the stage in `slot_` into KN/SN; the run's record is (ms_, hm_).
#define AKV_V_STEP(KC_, SC_, KN_, SN_, slot_, half_, ms_, hm_)                                                       \
    {                                                                                                                \
        const uint32_t fa_ = base + (uint32_t)(slot_) * P::F_BYTES + (uint32_t)(half_) * (vc::RUN * D) + c * 2;      \
        const uint32_t sa_ = base + P::S2_OFF + (uint32_t)(slot_) * P::S2_BYTES + (uint32_t)(g * TOK + (half_) * vc::RUN) * 4; \
        const uint32_t mla_ = base + P::ML_OFF + (uint32_t)((half_) * NML + ((ms_) < 0 ? 0 : (ms_))) * P::ML_BYTES + c; \
        if (__popc((hm_).x) <= 3) {                                                                                  \
            AKV_V_RUN_LEAN(KC_, SC_, KN_, SN_, fa_, sa_)                                                             \
            AKV_V_PATCH(KN_, fa_, mla_, (hm_).x, (hm_).y)                                                            \
        } else {                                                                                                     \
            AKV_V_RUN_FULL(KC_, SC_, KN_, SN_, fa_, sa_, mla_, (hm_).x, (hm_).y)                                     \
        }                                                                                                            \
    }
// Records of both runs of the stage in `slot_`: side slots and this head's {mid mask, low mask}.
#define AKV_V_RECORDS(slot_, msa_, hma_, msb_, hmb_)                                                  \
    {                                                                                                 \
        const uint32_t ra_ = base + P::REC_OFF + (uint32_t)((slot_) * 2) * P::REC_BYTES;              \
        msa_ = (int)lds32(ra_);                                                                       \
        hma_ = lds64(ra_ + 16 + g * 8);                                                               \
        msb_ = (int)lds32(ra_ + P::REC_BYTES);                                                        \
        hmb_ = lds64(ra_ + P::REC_BYTES + 16 + g * 8);                                                \
    }

template <int D, int G, int NS, int NML>
__global__ void __launch_bounds__(64 * G + 64) v_compute_kernel(const VParams p) {
    using P = VPlan<D, G, NS, NML>;
    constexpr int TOK = P::TOK;
    constexpr int NCH = 64 * G;                    // chain threads
    constexpr int HD = P::HD;                      // nibble row bytes
    static_assert(D == 128, "thread c of a head's two chain warps owns channels 2c, 2c+1");
    static_assert(NS <= vc::SCH, "the probability buffers are recycled assuming the ring is shorter than a chunk");
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const long long bh = blockIdx.x;               // (batch, KV head)
    const int n = p.n;
    const int nst = (n + TOK - 1) / TOK;
    const uint32_t base = smem_u32(smem);
    const uint32_t bar_full = base + P::BAR_OFF, bar_empty = bar_full + NS * 8, bar_ml = bar_empty + NS * 8;
    const uint32_t bar_sb = bar_ml + 2 * NML * 8;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full + s * 8, 2);          // one arrival per loader warp (+ the bytes they announce)
            mbar_init(bar_empty + s * 8, 2 * G);     // one arrival per chain warp
        }
        for (int s = 0; s < 2 * NML; ++s) mbar_init(bar_ml + s * 8, 2 * G);
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
#pragma unroll
        for (int u = 0; u < 32; ++u) kA[u] = kB[u] = 0;
#pragma unroll
        for (int v = 0; v < 8; ++v) sA[v] = sB[v] = make_uint4(0, 0, 0, 0);
        int slot = 0;              // slot of the stage whose first run is in kA / sA
        uint32_t phase = 0;
        bool alive = true;
        int ms0 = -1, ms1 = -1, msn0 = -1, msn1 = -1;      // side slots of this stage's / the next stage's runs
        uint2 hm0 = make_uint2(0, 0), hm1 = hm0, hmn0 = hm0, hmn1 = hm0;
        if (nsf > 0) {
            alive = mbar_wait(bar_full, 0);
            if (alive) {
                AKV_V_RECORDS(0, ms0, hm0, ms1, hm1)
                AKV_V_STEP(kB, sB, kA, sA, 0, 0, ms0, hm0)     // (a chain over zeros) fetch run 0 of stage 0
            }
        }
        for (int j = 0; j < nsf && alive; ++j) {
            // the next stage is looked at a run early, so that its records are in registers when they are needed
            const int nslot = slot + 1 == NS ? 0 : slot + 1;
            const uint32_t nphase = slot + 1 == NS ? phase ^ 1 : phase;
            const bool more = j + 1 < nsf;
            if (more) {
                alive = mbar_wait(bar_full + nslot * 8, nphase);
                if (!alive) break;
                AKV_V_RECORDS(nslot, msn0, hmn0, msn1, hmn1)
            }
            // first run of stage j while its second run is fetched
            AKV_V_STEP(kA, sA, kB, sB, slot, 1, ms1, hm1)
            // both runs of the stage are in registers: hand the slot and its side-ring slots back
            __syncwarp();
            if (lane == 0) {
                if (ms0 >= 0) mbar_arrive(bar_ml + (0 * NML + ms0) * 8);
                if (ms1 >= 0) mbar_arrive(bar_ml + (1 * NML + ms1) * 8);
                mbar_arrive(bar_empty + slot * 8);
            }
            // second run of stage j while the first run of stage j+1 is fetched
            if (more) {
                AKV_V_STEP(kB, sB, kA, sA, nslot, 0, msn0, hmn0)
            } else {
                AKV_V_RUN_NONE(kB, sB)
            }
            slot = nslot; phase = nphase;
            ms0 = msn0; hm0 = hmn0; ms1 = msn1; hm1 = hmn1;
        }
        if (tail > 0 && alive) {
            // last, partial stage: token by token straight from shared memory
            alive = mbar_wait(bar_full + slot * 8, phase);
            for (int t = 0; t < tail && alive; ++t) {
                const int half = t >> 5, u = t & 31;
                const uint32_t ra = base + P::REC_OFF + (uint32_t)(slot * 2 + half) * P::REC_BYTES;
                const int ms = (int)lds32(ra);
                const uint2 hm = lds64(ra + 16 + g * 8);
                uint32_t k = __byte_perm(lds16(base + (uint32_t)slot * P::F_BYTES + t * D + c * 2), 0x80u, 0x1404);
                if ((hm.x >> u) & 1u) {
                    const uint32_t mla = base + P::ML_OFF + (uint32_t)(half * NML + ms) * P::ML_BYTES + c;
                    const uint32_t mb = lds8(mla + u * HD);
                    const uint32_t lb = ((hm.y >> u) & 1u) ? lds8(mla + (32 + u) * HD) : 0x88u;
                    k = AKV_V_ASSEMBLE(lds16(base + (uint32_t)slot * P::F_BYTES + t * D + c * 2), mb, lb);
                }
                acc = hfma2_bits(k, lds32(base + P::S2_OFF + (uint32_t)slot * P::S2_BYTES + (g * TOK + t) * 4), acc);
            }
        }
        if (alive) reinterpret_cast<uint32_t*>(p.o)[((size_t)bh * G + g) * 64 + c] = acc;
        return;
    }

    // ---------------------------------------------------------------------- loader warps
    const int pt = tid - NCH, lane = pt & 31, pw = pt >> 5;
    const uint8_t* F = p.first8 + (size_t)bh * p.max_seq_len * D;
    const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * HD;
    const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * HD;
    const uint16_t* s_rows = p.s + (size_t)bh * G * p.s_last_dim;
    uint32_t A[G];
#pragma unroll
    for (int g = 0; g < G; ++g) A[g] = ((uint32_t)p.amin[bh * G + g] << 10) & 0xFFFFu;
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
    int slot = 0, ml_used = 0;          // stage slot; side-ring slots this warp has handed out so far
    uint32_t phase = 0;
    bool alive = true;
    if (pt == 0 && nst > 0) request_s(0);

    for (int j = 0; j < nst && alive; ++j) {
        if (j >= NS) alive = mbar_wait(bar_empty + slot * 8, phase ^ 1);   // stage j-NS has been consumed
        const int t0 = j * TOK;
        const int cnt = (n - t0) < TOK ? (n - t0) : TOK;
        const int c = j / vc::SCH, js = j - c * vc::SCH;
        if (js == 0) {   // entering chunk c: ask for the next one, make sure this one has landed
            if (pt == 0 && (c + 1) * vc::SCH < nst) request_s(c + 1);
            alive = alive && mbar_wait(bar_sb + (c % 3) * 8, (uint32_t)(c / 3) & 1u);
        }
        if (!alive) break;
        // decisions from the bit patterns (V_cache.cu:211,250-251): 16-bit wrap-around, signed compare
        uint32_t mm[G], lm[G];
        int ucode = 2;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const uint32_t sb = (pt < cnt) ? lds16(base + P::SB_OFF + (uint32_t)(c % 3) * P::SB_BYTES + g * P::SB_HEAD +
                                                   js * (TOK * 2) + pt * 2) : 0u;
            const int diff = (int)(int16_t)(uint16_t)(A[g] - sb);
            int code = p.reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
            if (pt >= cnt) code = 2;
            mm[g] = __ballot_sync(0xFFFFFFFFu, code < 2);
            lm[g] = __ballot_sync(0xFFFFFFFFu, code == 0);
            ucode = code < ucode ? code : ucode;
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(base + P::S2_OFF + (uint32_t)slot * P::S2_BYTES + (g * TOK + pt) * 4),
                         "r"(sb | (sb << 16)) : "memory");
        }
        const uint32_t umm = __ballot_sync(0xFFFFFFFFu, ucode < 2), ulm = __ballot_sync(0xFFFFFFFFu, ucode == 0);
        int ms = -1;
        uint32_t bytes = (pw == 0) ? (uint32_t)cnt * D : 0u;
        if (umm) {
            // the rows some head reads go to a slot of this warp's side ring
            ms = ml_used % NML;
            if (ml_used >= NML) alive = mbar_wait(bar_ml + (pw * NML + ms) * 8, ((ml_used / NML) & 1) ^ 1);
            ++ml_used;
            bytes += (uint32_t)HD * (__popc(umm) + __popc(ulm));
        }
        const uint32_t bar = bar_full + slot * 8;
        if (lane == 0) {
            const uint32_t ra = base + P::REC_OFF + (uint32_t)(slot * 2 + pw) * P::REC_BYTES;
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(ra), "r"(ms), "r"(umm), "r"(ulm), "r"(0) : "memory");
#pragma unroll
            for (int g = 0; g < G; ++g)
                asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(ra + 16 + g * 8), "r"(mm[g]), "r"(lm[g]) : "memory");
        }
        __syncwarp();
        if (!alive) break;
        if (lane == 0) {
            if (bytes) mbar_arrive_expect(bar, bytes);   // publishes this warp's stores, announces its copies
            else mbar_arrive(bar);
        }
        if (pt == 0) bulk_copy(base + (uint32_t)slot * P::F_BYTES, F + (size_t)t0 * D, (uint32_t)cnt * D, bar);
        if (umm) {
            const uint32_t dm = base + P::ML_OFF + (uint32_t)(pw * NML + ms) * P::ML_BYTES;
            const size_t src = (size_t)(t0 + pw * vc::RUN) * HD;
            // a run that reads a plane for all 32 tokens takes it as one 2 KB copy, otherwise row by row
            if (umm == 0xFFFFFFFFu) { if (lane == 0) bulk_copy(dm, M + src, vc::RUN * HD, bar); }
            else if (ucode < 2) bulk_copy(dm + lane * HD, M + src + (size_t)lane * HD, HD, bar);
            if (ulm == 0xFFFFFFFFu) { if (lane == 0) bulk_copy(dm + vc::RUN * HD, L + src, vc::RUN * HD, bar); }
            else if (ucode == 0) bulk_copy(dm + (vc::RUN + lane) * HD, L + src + (size_t)lane * HD, HD, bar);
        }
        if (++slot == NS) { slot = 0; phase ^= 1; }
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

template <int G, int NS, int NML>
static int launch_v_fast(const VParams& p, int BH, cudaStream_t st) {
    using K = VPlan<128, G, NS, NML>;
    static bool configured[64] = {false};   // the attribute is per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(v_compute_kernel<128, G, NS, NML>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)K::BYTES);
        if (e != cudaSuccess) return cuda_status(e, "v_cache_compute smem attribute");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    v_compute_kernel<128, G, NS, NML><<<BH, 64 * G + 64, K::BYTES, st>>>(p);
    return cuda_status(cudaGetLastError(), "v_cache_compute launch");
}

// P.V over n quantized tokens.  H = KV heads, group = query heads per KV head; s rows, amin bytes and output rows
// are per (batch, query head) with query head = KV head * group + g.
int launch_v_compute(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                     const uint8_t* amin, uint8_t* o, int bsz, int H, int group, int max_seq_len, int D,
                     int s_last_dim, int n, int reference, cudaStream_t st) {
    VParams p;
    p.first8 = first8; p.mid4 = mid4; p.last4 = last4;
    p.s = reinterpret_cast<const uint16_t*>(s);
    p.amin = amin;
    p.o = reinterpret_cast<uint16_t*>(o);
    p.max_seq_len = max_seq_len; p.D = D; p.s_last_dim = s_last_dim; p.n = n; p.reference = reference;
    p.group = group;
    const int BH = bsz * H;
    const bool fast = D == 128 && aligned16(first8) && aligned16(mid4) && aligned16(last4) &&
                      (n == 0 || (aligned16(s) && s_last_dim % 8 == 0 && ((n + 7) & ~7) <= s_last_dim)) &&
                      ((reinterpret_cast<uintptr_t>(o) & 3u) == 0);
    if (fast && group == 1) return launch_v_fast<1, 10, 2>(p, BH, st);
    if (fast && group == 2) return launch_v_fast<2, 10, 2>(p, BH, st);
    if (fast && group == 4) return launch_v_fast<4, 8, 2>(p, BH, st);
    long long total = (long long)BH * group * (D >> 1);
    long long want = (total + 127) / 128;
    int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
    if (grid < 1) grid = 1;
    v_compute_generic_kernel<<<grid, 128, 0, st>>>(p, BH * group);
    return cuda_status(cudaGetLastError(), "v_cache_compute launch");
}

// ================================================================== probe
// o_test[b,h,d] = sum_j |half((first_8[row_j][d] << 8) + 0x80)| * s_val[j], rows row_j = idx_j * K + j,
// accumulated in fp16 in j order (V_cache.cu:104-119).  All K row gathers are issued before the chain starts.
template <int KMAX>
__global__ void __launch_bounds__(128)
v_probe_kernel(const uint8_t* __restrict__ first8, const uint16_t* __restrict__ s_val,
               const int32_t* __restrict__ s_idx, uint16_t* __restrict__ out, int max_seq_len, int D, int K, int G) {
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
    v_probe_kernel<32><<<bsz * H * group, threads, 0, st>>>(first8, reinterpret_cast<const uint16_t*>(s_val),
                                                            reinterpret_cast<const int32_t*>(s_idx),
                                                            reinterpret_cast<uint16_t*>(out), max_seq_len, D, K, group);
    return cuda_status(cudaGetLastError(), "v_cache_test_compute launch");
}

}  // namespace akv

extern "C" int akv_device_error_flag(void) {
    // Non-zero once a bounded wait inside a kernel of this library gave up (never expected; the kernel then
    // returned early and its output is invalid).  Reading the flag synchronises the device.
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, akv::g_v_wait_gave_up, sizeof(v));
    if (e != cudaSuccess) return akv::cuda_status(e, "device_error_flag");
    return (int)v;
}
