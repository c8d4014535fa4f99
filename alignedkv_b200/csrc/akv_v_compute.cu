// Precision-aligned P.V over the quantized V tokens, and the magnitude probe that sets its threshold.
//
// Replaces the reference's v_cache_compute_kernel (extension/csrc/V_cache.cu:178-308) and
// v_cache_test_compute_kernel (V_cache.cu:90-123).  Outputs are bit-identical: each output channel is the fp16
// fused-multiply-add chain over tokens 0..n-1 in order, skipped nibble planes are replaced by the reference's
// constants (V_cache.cu:198-202,250-253).
//
// Design (B200): the exact token order leaves only B*H*D/2 independent chains - two warps per (batch, head) -
// and those warps are bound by their own instruction stream, so the kernel is organised around keeping that
// stream minimal and never letting it wait for memory.  One CTA per (batch, head), two roles:
//   chain warps (64 threads, thread c owns channels 2c, 2c+1): per token one 2-byte shared load, one byte permute
//     and one FMA; the loads and permutes of 32 tokens are issued before their dependent chain starts.
//   loader warps (64 threads, thread t owns token t of every 64-token stage): take the token's probability from a
//     shared buffer that is copied a whole 32-stage chunk ahead, decide from its bit pattern which of the token's 64-byte nibble
//     rows are needed, and issue 16-byte asynchronous copies: the 8 KB of high bytes into a deep ring of
//     high-byte-only stages, and - only for a run of 32 tokens in which some token needs a nibble plane - the
//     rows into a small side ring (rows that are not read get the reference's substitute constants).  Completion
//     is tracked by shared-memory mbarriers that the copies arrive on by themselves, so a loader never waits for
//     data, only for a free slot.
// Every wait is a bounded spin; a wait that gives up raises a flag the host can read (akv_device_error_flag).
#include "akv_common.cuh"

namespace akv {

namespace vc {
constexpr int TOK = 64;  // tokens per stage
}

struct VParams {
    const uint8_t* first8;
    const uint8_t* mid4;
    const uint8_t* last4;
    const uint16_t* s;
    const uint8_t* amin;
    uint16_t* o;
    int max_seq_len, D, s_last_dim, n, reference;
    int debug;
    unsigned long long* trace;   // experiments only
};

__device__ __forceinline__ void st_shared_row16(uint32_t a, uint32_t v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(a), "r"(v) : "memory");
}

// ---- shared-memory barriers (mbarrier) with bounded waits
static __device__ unsigned int g_v_wait_gave_up = 0;   // set when a bounded wait ran out (never expected)

__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(a) : "memory");
}
// arrives (without raising the pending count) once all earlier async copies of this thread have landed
__device__ __forceinline__ void mbar_arrive_on_copies(uint32_t a) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(a) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t a, uint32_t parity) {
    for (int spin = 0; spin < (1 << 22); ++spin) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
    }
    atomicOr(&g_v_wait_gave_up, 1u);
    return false;
}

// Shared-memory plan of one CTA.
//   F ring     NS stages of 64 tokens x D high bytes, filled by 16-byte async copies
//   meta       per stage: 64 probability words (both halves equal) and, per run of 32 tokens, the side-ring slot
//              that holds its nibble rows (-1: the run needs none)
//   side ring  per loader warp NML slots of [32 tokens x D/2 mid bytes][32 tokens x D/2 low bytes]
//   s chunks   per loader warp two buffers of 32 stages x 32 probabilities (that warp's tokens), copied a whole
//              chunk ahead so that no global-load latency sits on the staging loop
//   barriers   full / empty per stage, empty per side-ring slot, landed per probability buffer
template <int D, int NS, int NML>
struct VPlan {
    static constexpr int TOK = vc::TOK;
    static constexpr int HD = D / 2;
    static constexpr int F_BYTES = TOK * D;
    static constexpr int META_OFF = NS * F_BYTES;
    static constexpr int META_BYTES = TOK * 4 + 32;   // + per run of 32 tokens: side slot, mid mask, low mask, pad
    static constexpr int ML_OFF = META_OFF + NS * META_BYTES;
    static constexpr int ML_BYTES = 32 * HD * 2;
    static constexpr int SCH = 32;                               // stages per probability chunk
    static constexpr int S_OFF = ML_OFF + 2 * NML * ML_BYTES;    // per loader warp: 2 chunks x 32 stages x 32 fp16
    static constexpr int S_BYTES = 2 * SCH * 32 * 2;
    static constexpr int BAR_OFF = S_OFF + 2 * S_BYTES;
    static constexpr int BYTES = BAR_OFF + (2 * NS + 2 * NML + 4) * 8;
};

template <int NS, int NML, int D>
__global__ void __launch_bounds__(D) v_compute_kernel(const VParams p) {
    using P = VPlan<D, NS, NML>;
    constexpr int TOK = P::TOK;
    constexpr int NC = D / 2;                      // chain threads; thread c owns channels 2c, 2c+1
    constexpr int NL = TOK;                        // loader threads; thread t owns token t of a stage
    constexpr int HD = P::HD;                      // nibble row bytes
    constexpr int F_OPS = P::F_BYTES / 16 / NL;    // 16-byte copies per loader thread for the high-byte plane
    constexpr int ROW_OPS = HD / 16;               // 16-byte copies per nibble row
    static_assert(NC == 64 && NL == 64, "two chain warps and two loader warps");
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const long long bh = blockIdx.x;
    const int n = p.n;
    const int nst = (n + TOK - 1) / TOK;
    const uint32_t base = smem_u32(smem);
    const uint32_t bar_full = base + P::BAR_OFF, bar_empty = bar_full + NS * 8, bar_ml = bar_empty + NS * 8;
    const uint32_t bar_s = bar_ml + 2 * NML * 8;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full + s * 8, 2 * NL);    // per loader thread: one arrival by its copies, one by itself
            mbar_init(bar_empty + s * 8, NC);
        }
        for (int s = 0; s < 2 * NML; ++s) mbar_init(bar_ml + s * 8, NC);
        for (int s = 0; s < 4; ++s) mbar_init(bar_s + s * 8, 32);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    if (tid < NC) {
        // ------------------------------------------------------------------ chain warps
        uint32_t acc = 0;
        int slot = 0;
        uint32_t phase = 0;
        bool alive = true;
        // One run of 32 tokens: K_[u] holds k~ = [0x80, f_even, 0x80, f_odd] of token u; tokens whose bit is set in
        // the run's mid mask take their low bytes from the side ring instead (warp-uniform, rare branch).
#define AKV_V_RUN(K_, S_, MM_, LM_, MLA_)                                                              \
        _Pragma("unroll") for (int v_ = 0; v_ < 8; ++v_) {                                             \
            _Pragma("unroll") for (int w_ = 0; w_ < 4; ++w_) {                                         \
                const int u_ = 4 * v_ + w_;                                                            \
                uint32_t k_ = K_[u_];                                                                  \
                if ((MM_ >> u_) & 1u) {                                                                \
                    const uint32_t mb_ = lds8(MLA_ + u_ * HD);                                         \
                    const uint32_t lb_ = ((LM_ >> u_) & 1u) ? lds8(MLA_ + 32 * HD + u_ * HD) : 0x88u;  \
                    const uint32_t lo_e_ = (mb_ & 0xF0u) | (lb_ >> 4);                                 \
                    const uint32_t lo_o_ = ((mb_ << 4) & 0xF0u) | (lb_ & 0x0Fu);                       \
                    k_ = (k_ & 0xFF00FF00u) | lo_e_ | (lo_o_ << 16);                                   \
                }                                                                                      \
                const uint32_t s_ = (w_ == 0) ? S_[v_].x : (w_ == 1) ? S_[v_].y : (w_ == 2) ? S_[v_].z : S_[v_].w; \
                acc = hfma2_bits(k_, s_, acc);                                                         \
            }                                                                                          \
        }
        // The common run: no token reads a nibble plane, so the chain is 32 back-to-back FMAs.
#define AKV_V_RUN_LEAN(K_, S_)                                   \
        _Pragma("unroll") for (int v_ = 0; v_ < 8; ++v_) {       \
            acc = hfma2_bits(K_[4 * v_], S_[v_].x, acc);         \
            acc = hfma2_bits(K_[4 * v_ + 1], S_[v_].y, acc);     \
            acc = hfma2_bits(K_[4 * v_ + 2], S_[v_].z, acc);     \
            acc = hfma2_bits(K_[4 * v_ + 3], S_[v_].w, acc);     \
        }
        for (int i = 0; i < nst && alive; ++i) {
            if (p.trace && bh == 0 && tid == 0) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); p.trace[i * 4 + 0] = t; }
            alive = mbar_wait(bar_full + slot * 8, phase);
            if (p.trace && bh == 0 && tid == 0) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); p.trace[i * 4 + 1] = t; }
            const uint32_t fa = base + (uint32_t)slot * P::F_BYTES + tid * 2;            // + t * D
            const uint32_t ma = base + P::META_OFF + (uint32_t)slot * P::META_BYTES;     // s2 words, then run records
            const int cnt = (n - i * TOK) < TOK ? (n - i * TOK) : TOK;
            const uint4 r0 = lds128(ma + TOK * 4), r1 = lds128(ma + TOK * 4 + 16);       // {slot, mid mask, low mask, -}
            const uint32_t mla0 = base + P::ML_OFF + (uint32_t)(0 * NML + (int)r0.x) * P::ML_BYTES + tid;
            const uint32_t mla1 = base + P::ML_OFF + (uint32_t)(1 * NML + (int)r1.x) * P::ML_BYTES + tid;
            if (p.debug & 1) {
            } else if (cnt == TOK) {
                uint32_t k0[32], k1[32];
                uint4 s0[8], s1[8];
#pragma unroll
                for (int u = 0; u < 32; ++u) k0[u] = lds16(fa + u * D);
#pragma unroll
                for (int v = 0; v < 8; ++v) s0[v] = lds128(ma + 4 * v * 4);
#pragma unroll
                for (int u = 0; u < 32; ++u) k1[u] = lds16(fa + (32 + u) * D);     // second run's loads are in
#pragma unroll
                for (int v = 0; v < 8; ++v) s1[v] = lds128(ma + (32 + 4 * v) * 4); // flight during the first chain
#pragma unroll
                for (int u = 0; u < 32; ++u) k0[u] = __byte_perm(k0[u], 0x80u, 0x1404);
                if (r0.y == 0) { AKV_V_RUN_LEAN(k0, s0) } else { AKV_V_RUN(k0, s0, r0.y, r0.z, mla0) }
#pragma unroll
                for (int u = 0; u < 32; ++u) k1[u] = __byte_perm(k1[u], 0x80u, 0x1404);
                if (r1.y == 0) { AKV_V_RUN_LEAN(k1, s1) } else { AKV_V_RUN(k1, s1, r1.y, r1.z, mla1) }
            } else {
                // last, partial stage: token by token; rows past cnt hold stale bytes and must not be touched
                for (int t = 0; t < cnt; ++t) {
                    const uint4 r = (t < 32) ? r0 : r1;
                    const uint32_t mla = (t < 32) ? mla0 : mla1;
                    const int u = t & 31;
                    uint32_t k = __byte_perm(lds16(fa + t * D), 0x80u, 0x1404);
                    if ((r.y >> u) & 1u) {
                        const uint32_t mb = lds8(mla + u * HD);
                        const uint32_t lb = ((r.z >> u) & 1u) ? lds8(mla + 32 * HD + u * HD) : 0x88u;
                        k = (k & 0xFF00FF00u) | ((mb & 0xF0u) | (lb >> 4)) | ((((mb << 4) & 0xF0u) | (lb & 0x0Fu)) << 16);
                    }
                    acc = hfma2_bits(k, lds32(ma + t * 4), acc);
                }
            }
            if ((int)r0.x >= 0) mbar_arrive(bar_ml + (0 * NML + (int)r0.x) * 8);   // side-ring slots may be refilled
            if ((int)r1.x >= 0) mbar_arrive(bar_ml + (1 * NML + (int)r1.x) * 8);
            if (p.trace && bh == 0 && tid == 0) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); p.trace[i * 4 + 2] = t; }
            mbar_arrive(bar_empty + slot * 8);
            if (++slot == NS) { slot = 0; phase ^= 1; }
        }
#undef AKV_V_RUN
#undef AKV_V_RUN_LEAN
        reinterpret_cast<uint32_t*>(p.o)[(size_t)bh * NC + tid] = acc;
        return;
    }

    // ---------------------------------------------------------------------- loader warps
    const int pt = tid - NC, lane = pt & 31, pw = pt >> 5;
    const uint8_t* F = p.first8 + (size_t)bh * p.max_seq_len * D;
    const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * HD;
    const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * HD;
    const uint16_t* s_row = p.s + (size_t)bh * p.s_last_dim;
    const uint32_t A = ((uint32_t)p.amin[bh] << 10) & 0xFFFFu;
    // Probability chunk c (stages 32c .. 32c+31, this warp's 32 tokens of each) -> this warp's buffer c & 1.
    // 4 x 16 bytes per stage; the barrier of the buffer completes when every lane's copies have landed.
    const uint32_t sbuf = base + P::S_OFF + (uint32_t)pw * P::S_BYTES;
    auto request_s = [&](int c) {
        const uint32_t dst = sbuf + (uint32_t)(c & 1) * (P::SCH * 64);
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int op = it * 32 + lane;              // 128 pieces: stage (op >> 2), 8 tokens (op & 3)
            const int t = (c * P::SCH + (op >> 2)) * TOK + pw * 32 + (op & 3) * 8;
            if (t < n) cp_async16(dst + (op >> 2) * 64 + (op & 3) * 16, s_row + t);
        }
        mbar_arrive_on_copies(bar_s + (pw * 2 + (c & 1)) * 8);
    };
    int slot = 0, ml_used = 0;          // stage slot; side-ring slots this warp has handed out so far
    uint32_t phase = 0;
    bool alive = true;

    auto stage = [&](int j) {
        if (j >= NS) alive = alive && mbar_wait(bar_empty + slot * 8, phase ^ 1);   // stage j-NS has been consumed
        const uint32_t st = base + (uint32_t)slot * P::F_BYTES;
        const int t0 = j * TOK;
        const int cnt = (n - t0) < TOK ? (n - t0) : TOK;
        const int fbytes = cnt * D;  // high-byte plane: cnt*D contiguous bytes
        if (!(p.debug & 2)) {
#pragma unroll
            for (int it = 0; it < F_OPS; ++it) {
                const int off = (it * NL + pt) << 4;
                if (off < fbytes) cp_async16(st + off, F + (size_t)t0 * D + off);
            }
        }
        const int c = j / P::SCH, js = j - c * P::SCH;
        if (js == 0) {   // entering chunk c: ask for the next one, make sure this one has landed
            if ((c + 1) * P::SCH < nst) request_s(c + 1);
            alive = alive && mbar_wait(bar_s + (pw * 2 + (c & 1)) * 8, (uint32_t)(c >> 1) & 1u);
        }
        const uint32_t sb = (pt < cnt) ? lds16(sbuf + (uint32_t)(c & 1) * (P::SCH * 64) + js * 64 + lane * 2) : 0u;
        // decision from the bit patterns (V_cache.cu:211,250-251): 16-bit wrap-around, signed compare
        const int diff = (int)(int16_t)(uint16_t)(A - sb);
        int code = p.reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
        if (pt >= cnt) code = 2;
        // which of this warp's 32 tokens read the mid plane / the low plane
        const uint32_t mmask = __ballot_sync(0xFFFFFFFFu, code < 2), lmask = __ballot_sync(0xFFFFFFFFu, code == 0);
        const uint32_t ma = base + P::META_OFF + (uint32_t)slot * P::META_BYTES;
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(ma + pt * 4), "r"(sb | (sb << 16)) : "memory");
        int ms = -1;
        if (mmask) {
            // their 64-byte rows go to a slot of this warp's side ring; rows of other tokens are not touched
            ms = ml_used % NML;
            if (ml_used >= NML) alive = alive && mbar_wait(bar_ml + (pw * NML + ms) * 8, ((ml_used / NML) & 1) ^ 1);
            ++ml_used;
            const size_t src = (size_t)(t0 + pt) * HD;
            const uint32_t dm = base + P::ML_OFF + (uint32_t)(pw * NML + ms) * P::ML_BYTES + lane * HD;
            const uint32_t dl = dm + 32 * HD;
            if (code < 2) {
#pragma unroll
                for (int v = 0; v < ROW_OPS; ++v) cp_async16(dm + v * 16, M + src + v * 16);
            }
            if (code == 0) {
#pragma unroll
                for (int v = 0; v < ROW_OPS; ++v) cp_async16(dl + v * 16, L + src + v * 16);
            }
        }
        if (lane == 0)
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(ma + TOK * 4 + pw * 16), "r"(ms), "r"(mmask),
                         "r"(lmask), "r"(0) : "memory");
        if (p.trace && bh == 0 && pt == 0) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); p.trace[j * 4 + 3] = t; }
        mbar_arrive_on_copies(bar_full + slot * 8);   // fires when this thread's copies (all of them) have landed
        mbar_arrive(bar_full + slot * 8);             // publishes this thread's plain stores
        if (++slot == NS) { slot = 0; phase ^= 1; }
    };

    request_s(0);
    for (int j = 0; j < nst && alive; ++j) stage(j);
    cp_async_commit();
    cp_async_wait<0>();   // this thread's copies must have landed before its shared memory goes away
}

// Any even head_dim: one thread per channel pair, planes read straight from global memory.
__global__ void __launch_bounds__(128)
v_compute_generic_kernel(const VParams p, int bh_count) {
    const int hd = p.D >> 1;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)bh_count * hd;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % hd);
        const long long bh = i / hd;
        const uint8_t* F = p.first8 + (size_t)bh * p.max_seq_len * p.D;
        const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * hd;
        const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * hd;
        const uint16_t* s_row = p.s + (size_t)bh * p.s_last_dim;
        const uint32_t A = ((uint32_t)p.amin[bh] << 10) & 0xFFFFu;
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
        reinterpret_cast<uint32_t*>(p.o)[(size_t)bh * hd + c] = acc;
    }
}

template <int NS, int NML, int D>
static int launch_v_fast(const VParams& p, int BH, cudaStream_t st) {
    size_t smem = (size_t)VPlan<D, NS, NML>::BYTES;
    cudaError_t e = cudaFuncSetAttribute(v_compute_kernel<NS, NML, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return cuda_status(e, "v_cache_compute smem attribute");
    v_compute_kernel<NS, NML, D><<<BH, D, smem, st>>>(p);
    return cuda_status(cudaGetLastError(), "v_cache_compute launch");
}

int launch_v_compute(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                     const uint8_t* amin, uint8_t* o, int bsz, int H, int max_seq_len, int D, int s_last_dim,
                     int n, int reference, cudaStream_t st) {
    VParams p;
    p.first8 = first8; p.mid4 = mid4; p.last4 = last4;
    p.s = reinterpret_cast<const uint16_t*>(s);
    p.amin = amin;
    p.o = reinterpret_cast<uint16_t*>(o);
    p.max_seq_len = max_seq_len; p.D = D; p.s_last_dim = s_last_dim; p.n = n; p.reference = reference;
    p.debug = tuning().debug;
    p.trace = reinterpret_cast<unsigned long long*>(((unsigned long long)(unsigned)tuning().trace_hi << 32) | (unsigned)tuning().trace_lo);
    const int BH = bsz * H;
    const bool fast = D == 128 && aligned16(first8) && aligned16(mid4) && aligned16(last4) &&
                      (n == 0 || (aligned16(s) && s_last_dim % 8 == 0)) &&
                      ((reinterpret_cast<uintptr_t>(o) & 3u) == 0);
    if (fast) {
        const int stages = tuning().v_stages;
        if (stages == 4) return launch_v_fast<6, 2, 128>(p, BH, st);
        if (stages == 8) return launch_v_fast<8, 2, 128>(p, BH, st);
        return launch_v_fast<10, 2, 128>(p, BH, st);
    }
    long long total = (long long)BH * (D >> 1);
    long long want = (total + 127) / 128;
    int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
    if (grid < 1) grid = 1;
    v_compute_generic_kernel<<<grid, 128, 0, st>>>(p, BH);
    return cuda_status(cudaGetLastError(), "v_cache_compute launch");
}

// ================================================================== probe
// o_test[b,h,d] = sum_j |half((first_8[row_j][d] << 8) + 0x80)| * s_val[j], rows row_j = idx_j * K + j,
// accumulated in fp16 in j order (V_cache.cu:104-119).  All K row gathers are issued before the chain starts.
template <int KMAX>
__global__ void __launch_bounds__(128)
v_probe_kernel(const uint8_t* __restrict__ first8, const uint16_t* __restrict__ s_val,
               const int32_t* __restrict__ s_idx, uint16_t* __restrict__ out, int max_seq_len, int D, int K) {
    const long long bh = blockIdx.x;
    const uint8_t* F = first8 + (size_t)bh * max_seq_len * D;
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
                   int max_seq_len, int D, int K, cudaStream_t st) {
    int threads = (D >> 1) < 128 ? (((D >> 1) + 31) / 32) * 32 : 128;
    v_probe_kernel<32><<<bsz * H, threads, 0, st>>>(first8, reinterpret_cast<const uint16_t*>(s_val),
                                                    reinterpret_cast<const int32_t*>(s_idx),
                                                    reinterpret_cast<uint16_t*>(out), max_seq_len, D, K);
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
