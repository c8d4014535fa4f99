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
//     register pipeline fetched four stages ahead, decide from its bit pattern which of the token's 64-byte nibble
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
//   barriers   full / empty per stage, empty per side-ring slot
template <int D, int NS, int NML>
struct VPlan {
    static constexpr int TOK = vc::TOK;
    static constexpr int HD = D / 2;
    static constexpr int F_BYTES = TOK * D;
    static constexpr int META_OFF = NS * F_BYTES;
    static constexpr int META_BYTES = TOK * 4 + 16;
    static constexpr int ML_OFF = META_OFF + NS * META_BYTES;
    static constexpr int ML_BYTES = 32 * HD * 2;
    static constexpr int BAR_OFF = ML_OFF + 2 * NML * ML_BYTES;
    static constexpr int BYTES = BAR_OFF + (2 * NS + 2 * NML) * 8;
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

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full + s * 8, 2 * NL);    // per loader thread: one arrival by its copies, one by itself
            mbar_init(bar_empty + s * 8, NC);
        }
        for (int s = 0; s < 2 * NML; ++s) mbar_init(bar_ml + s * 8, NC);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    if (tid < NC) {
        // ------------------------------------------------------------------ chain warps
        uint32_t acc = 0;
        int slot = 0;
        uint32_t phase = 0;
        bool alive = true;
        for (int i = 0; i < nst && alive; ++i) {
            alive = mbar_wait(bar_full + slot * 8, phase);
            const uint32_t fa = base + (uint32_t)slot * P::F_BYTES + tid * 2;            // + t * D
            const uint32_t ma = base + P::META_OFF + (uint32_t)slot * P::META_BYTES;     // s2 words, then 2 slot ids
            const int cnt = (n - i * TOK) < TOK ? (n - i * TOK) : TOK;
            if (!(p.debug & 1)) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const int tb = hf * 32;
                    const int ms = (int)lds32(ma + TOK * 4 + hf * 4);
                    if (ms < 0) {
                        // 32 tokens, high byte only: k~ = [0x80, f_even, 0x80, f_odd]
                        uint32_t f[32];
                        uint4 sv[8];
#pragma unroll
                        for (int u = 0; u < 32; ++u) f[u] = lds16(fa + (tb + u) * D);
#pragma unroll
                        for (int v = 0; v < 8; ++v) sv[v] = lds128(ma + (tb + 4 * v) * 4);
#pragma unroll
                        for (int u = 0; u < 32; ++u) f[u] = __byte_perm(f[u], 0x80u, 0x1404);
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            acc = hfma2_bits(f[4 * v], sv[v].x, acc);
                            acc = hfma2_bits(f[4 * v + 1], sv[v].y, acc);
                            acc = hfma2_bits(f[4 * v + 2], sv[v].z, acc);
                            acc = hfma2_bits(f[4 * v + 3], sv[v].w, acc);
                        }
                    } else {
                        const uint32_t mla = base + P::ML_OFF + (uint32_t)(hf * NML + ms) * P::ML_BYTES + tid;
                        const int end = cnt < tb + 32 ? cnt : tb + 32;
                        for (int t0 = tb; t0 < end; t0 += 8) {
                            uint32_t f[8], mb[8], lb[8], s2[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int t = t0 + u;   // rows past the stage's tokens hold stale bytes; not used
                                f[u] = lds16(fa + t * D);
                                mb[u] = lds8(mla + (t - tb) * HD);
                                lb[u] = lds8(mla + 32 * HD + (t - tb) * HD);
                                s2[u] = lds32(ma + t * 4);
                            }
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                if (t0 + u < end) {
                                    const uint32_t lo_e = (mb[u] & 0xF0u) | (lb[u] >> 4);            // even channel
                                    const uint32_t lo_o = ((mb[u] << 4) & 0xF0u) | (lb[u] & 0x0Fu);  // odd channel
                                    acc = hfma2_bits(__byte_perm(f[u], lo_e | (lo_o << 8), 0x1504), s2[u], acc);
                                }
                            }
                        }
                        mbar_arrive(bar_ml + (hf * NML + ms) * 8);   // the side-ring slot may be refilled
                    }
                }
            }
            mbar_arrive(bar_empty + slot * 8);
            if (++slot == NS) { slot = 0; phase ^= 1; }
        }
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
    auto load_s = [&](int j) -> uint32_t {   // probability of this thread's token of stage j (0 beyond n)
        const int t = j * TOK + pt;
        return (t < n) ? (uint32_t)__ldg(s_row + t) : 0u;
    };
    int slot = 0, ml_used = 0;          // stage slot; side-ring slots this warp has handed out so far
    uint32_t phase = 0;
    bool alive = true;

    auto stage = [&](int j, uint32_t sb) {
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
        // decision from the bit patterns (V_cache.cu:211,250-251): 16-bit wrap-around, signed compare
        const int diff = (int)(int16_t)(uint16_t)(A - sb);
        int code = p.reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
        if (pt >= cnt) code = 2;
        // this warp's 32 tokens are "lean" when all of them exist and none reads a nibble plane
        const bool lean = __all_sync(0xFFFFFFFFu, code == 2) && (t0 + pw * 32 + 32 <= n);
        const uint32_t ma = base + P::META_OFF + (uint32_t)slot * P::META_BYTES;
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(ma + pt * 4), "r"(sb | (sb << 16)) : "memory");
        int ms = -1;
        if (!lean) {
            ms = ml_used % NML;
            if (ml_used >= NML) alive = alive && mbar_wait(bar_ml + (pw * NML + ms) * 8, ((ml_used / NML) & 1) ^ 1);
            ++ml_used;
            // rows the rule reads are fetched; the others get the reference's substitute bytes (mid 0x88 / low 0x00
            // when neither is read, low 0x88 when only mid is read), so the consumer has no per-token branch
            const size_t src = (size_t)(t0 + pt) * HD;
            const uint32_t dm = base + P::ML_OFF + (uint32_t)(pw * NML + ms) * P::ML_BYTES + lane * HD;
            const uint32_t dl = dm + 32 * HD;
#pragma unroll
            for (int v = 0; v < ROW_OPS; ++v) {
                if (code < 2) cp_async16(dm + v * 16, M + src + v * 16);
                else st_shared_row16(dm + v * 16, 0x88888888u);
                if (code == 0) cp_async16(dl + v * 16, L + src + v * 16);
                else st_shared_row16(dl + v * 16, code == 1 ? 0x88888888u : 0u);
            }
        }
        if (lane == 0) asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(ma + TOK * 4 + pw * 4), "r"(ms) : "memory");
        mbar_arrive_on_copies(bar_full + slot * 8);   // fires when this thread's copies (all of them) have landed
        mbar_arrive(bar_full + slot * 8);             // publishes this thread's plain stores
        if (++slot == NS) { slot = 0; phase ^= 1; }
    };

    uint32_t s0 = load_s(0), s1 = load_s(1), s2 = load_s(2), s3 = load_s(3);
    for (int j0 = 0; j0 < nst && alive; j0 += 4) {
        stage(j0, s0);
        s0 = load_s(j0 + 4);
        if (j0 + 1 < nst) { stage(j0 + 1, s1); s1 = load_s(j0 + 5); }
        if (j0 + 2 < nst) { stage(j0 + 2, s2); s2 = load_s(j0 + 6); }
        if (j0 + 3 < nst) { stage(j0 + 3, s3); s3 = load_s(j0 + 7); }
    }
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
