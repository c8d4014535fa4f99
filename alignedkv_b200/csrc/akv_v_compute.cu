// Precision-aligned P.V over the quantized V tokens, and the magnitude probe that sets its threshold.
//
// Replaces the reference's v_cache_compute_kernel (extension/csrc/V_cache.cu:178-308) and
// v_cache_test_compute_kernel (V_cache.cu:90-123).  Outputs are bit-identical: each output channel is the fp16
// fused-multiply-add chain over tokens 0..n-1 in order, skipped nibble planes are replaced by the reference's
// constants (V_cache.cu:198-202,250-253).
//
// Design (B200): one CTA of 64 threads per (batch, head) - thread c owns channels 2c, 2c+1 and their serial
// chains.  What the reference leaves latency-bound (every token waits for four dependent byte loads) is
// decoupled here: the CTA streams 64-token stages of the high-byte plane through a deep ring of shared memory
// with 16-byte asynchronous copies, thread t decides from the probability bits of token t whether that token's
// 64-byte mid / low rows are fetched at all, and the consumer loop runs from shared memory at FMA latency.
// Runs of 8 tokens that need no nibble plane (the common case) take a 3-instruction-per-token path.
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
    int pf_dist;   // L2 prefetch distance in stages (0 = off)
    int debug;
};

__device__ __forceinline__ void st_shared_row16(uint32_t a, uint32_t v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(a), "r"(v) : "memory");
}
// Named barriers (ids 1..15): producers and consumers hand stages over without spinning.
__device__ __forceinline__ void bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(int id, int count) {
    asm volatile("bar.arrive %0, %1;\n" ::"r"(id), "r"(count) : "memory");
}

// Shared-memory plan of one CTA.
//   raw ring   RAW stages of [F: 64*D][M: 64*D/2][L: 64*D/2]                 filled by 16-byte async copies
//   ready ring RDY stages of [kv: 64 tokens x D/2 fp16x2 words][s2: 64 words]   filled by the unpackers
//   s ring     8 chunks of 64 probabilities, copied SA stages before the stage that needs them, so that the
//              plane-read decision of a token never waits for a global load
//   meta       per raw stage: the 64 probability words and two "lean" flags (one per 32 tokens)
template <int D, int RAW, int RDY>
struct VPlan {
    static constexpr int TOK = vc::TOK;
    static constexpr int HD = D / 2;
    static constexpr int F_BYTES = TOK * D;
    static constexpr int N_BYTES = TOK * HD;
    static constexpr int RAW_BYTES = F_BYTES + 2 * N_BYTES;
    static constexpr int KV_BYTES = TOK * HD * 4;
    static constexpr int RDY_BYTES = KV_BYTES + TOK * 4;
    static constexpr int RDY_OFF = RAW * RAW_BYTES;
    static constexpr int SRING = 8;
    static constexpr int S_OFF = RDY_OFF + RDY * RDY_BYTES;
    static constexpr int META_OFF = S_OFF + SRING * TOK * 2;
    static constexpr int META_BYTES = TOK * 4 + 16;
    static constexpr int BYTES = META_OFF + RAW * META_BYTES;
};

// Threads [0, D/2): chain warps - thread c owns channels 2c, 2c+1 and runs their serial fp16 chains from the
// ready ring (per token: one shared load and one FMA, nothing else).
// Threads [D/2, D/2 + 32*NSTG): staging warps - they issue the async copies of a stage, decide from the
// probability bits of each token which nibble rows are fetched (staging thread t < 64 owns token t), and
// reassemble landed stages into fp16x2 words for the chain warps.
template <int RAW, int RDY, int D, int NSTG>
__global__ void __launch_bounds__(D / 2 + 32 * NSTG) v_compute_kernel(const VParams p) {
    using P = VPlan<D, RAW, RDY>;
    constexpr int TOK = P::TOK;
    constexpr int NC = D / 2;                      // chain threads
    constexpr int NS = 32 * NSTG;                  // staging threads
    constexpr int NT = NC + NS;
    constexpr int HD = P::HD;
    constexpr int F_OPS = (P::F_BYTES / 16 + NS - 1) / NS;   // 16-byte copies per staging thread, high-byte plane
    constexpr int ROW_OPS = HD / 16;                          // 16-byte copies per nibble row
    constexpr int ITEMS = TOK * (D / 8) / NS;                 // (token, 8-channel) pieces per staging thread
    constexpr int SA = 4;                          // probability chunks run SA stages ahead of the plane copies
    static_assert(NC == TOK, "one chain thread per staged token is assumed by the ready-stage layout");
    static_assert(NS >= TOK && (TOK * (D / 8)) % NS == 0, "staging thread count");
    static_assert(SA >= RAW - 1 && SA + RAW <= P::SRING, "s ring depth");
    static_assert(RDY >= 2 && 2 * RDY + 1 <= 15, "named barriers");
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const long long bh = blockIdx.x;
    const int n = p.n;
    const int nst = (n + TOK - 1) / TOK;
    const uint32_t base = smem_u32(smem);
    // barrier ids: 1 = staging warps only; 2+2r = ready slot r full; 3+2r = ready slot r empty

    if (tid < NC) {
        // ------------------------------------------------------------------ chain warps
        const int c = tid;
        uint32_t acc = 0;
        for (int i = 0; i < nst; ++i) {
            const int slot = i % RDY;
            bar_sync(2 + 2 * slot, NT);
            const uint32_t ra = base + P::RDY_OFF + (uint32_t)slot * P::RDY_BYTES;
            const uint32_t kva = ra + c * 4;              // + t * NC * 4
            const uint32_t sa = ra + P::KV_BYTES;         // + t * 4 (probability in both halves)
            const int cnt = (n - i * TOK) < TOK ? (n - i * TOK) : TOK;
            if (cnt == TOK && !(p.debug & 1)) {
                uint32_t cur[16], nxt[16];
                uint4 cs[4], ns[4];
#pragma unroll
                for (int u = 0; u < 16; ++u) cur[u] = lds32(kva + u * NC * 4);
#pragma unroll
                for (int v = 0; v < 4; ++v) cs[v] = lds128(sa + v * 16);
#pragma unroll
                for (int b = 0; b < TOK / 16; ++b) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        if (b + 1 < TOK / 16) {   // next batch's loads ride between the dependent FMAs
                            ns[v] = lds128(sa + ((b + 1) * 4 + v) * 16);
#pragma unroll
                            for (int w = 0; w < 4; ++w) nxt[4 * v + w] = lds32(kva + ((b + 1) * 16 + 4 * v + w) * NC * 4);
                        }
                        acc = hfma2_bits(cur[4 * v], cs[v].x, acc);
                        acc = hfma2_bits(cur[4 * v + 1], cs[v].y, acc);
                        acc = hfma2_bits(cur[4 * v + 2], cs[v].z, acc);
                        acc = hfma2_bits(cur[4 * v + 3], cs[v].w, acc);
                    }
#pragma unroll
                    for (int u = 0; u < 16; ++u) cur[u] = nxt[u];
#pragma unroll
                    for (int v = 0; v < 4; ++v) cs[v] = ns[v];
                }
            } else if (!(p.debug & 1)) {
                for (int t = 0; t < cnt; ++t) acc = hfma2_bits(lds32(kva + t * NC * 4), lds32(sa + t * 4), acc);
            }
            if (i + RDY < nst) bar_arrive(3 + 2 * slot, NT);   // hand the slot back if it is needed again
        }
        reinterpret_cast<uint32_t*>(p.o)[(size_t)bh * NC + c] = acc;
        return;
    }

    // ---------------------------------------------------------------------- staging warps
    const int pt = tid - NC;                     // staging thread index; pt < 64 owns token pt of every stage
    const uint8_t* F = p.first8 + (size_t)bh * p.max_seq_len * D;
    const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * HD;
    const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * HD;
    const uint16_t* s_row = p.s + (size_t)bh * p.s_last_dim;
    const uint32_t A = ((uint32_t)p.amin[bh] << 10) & 0xFFFFu;

    // chunk of 64 probabilities for stage j -> s ring (8 threads x 16 bytes); beyond n nothing is copied and
    // the decision code below treats those tokens as absent
    auto stage_s = [&](int j) {
        const int t0 = j * TOK + pt * 8;
        if (pt < 8 && t0 < n)
            cp_async16(base + P::S_OFF + (uint32_t)(j % P::SRING) * (TOK * 2) + pt * 16, s_row + t0);
    };

    auto issue = [&](int j, int rslot) {
        const uint32_t st = base + (uint32_t)rslot * P::RAW_BYTES;
        const int t0 = j * TOK;
        const int cnt = (n - t0) < TOK ? (n - t0) : TOK;
        const int fbytes = cnt * D;  // high-byte plane: cnt*D contiguous bytes
        if (!(p.debug & 2)) {
#pragma unroll
            for (int it = 0; it < F_OPS; ++it) {
                const int off = (it * NS + pt) << 4;
                if (off < fbytes) cp_async16(st + off, F + (size_t)t0 * D + off);
            }
        }
        stage_s(j + SA);
        if (pt < TOK) {
            const uint32_t sb = (pt < cnt) ? lds16(base + P::S_OFF + (uint32_t)(j % P::SRING) * (TOK * 2) + pt * 2) : 0u;
            // decision from the bit patterns (V_cache.cu:211,250-251): 16-bit wrap-around, signed compare
            const int diff = (int)(int16_t)(uint16_t)(A - sb);
            int code = p.reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
            if (pt >= cnt) code = 2;
            // 32 tokens are "lean" when all of them exist and none reads a nibble plane
            const bool lean = __all_sync(0xFFFFFFFFu, code == 2) && (t0 + (pt & 32) + 32 <= n);
            const uint32_t ma = base + P::META_OFF + (uint32_t)rslot * P::META_BYTES;
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(ma + pt * 4), "r"(sb | (sb << 16)) : "memory");
            if ((pt & 31) == 0)
                asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(ma + TOK * 4 + (pt >> 5) * 4), "r"((uint32_t)lean)
                             : "memory");
            if (!lean) {
                // rows the rule reads are fetched; the others get the reference's substitute bytes (mid 0x88 /
                // low 0x00 when neither is read, low 0x88 when only mid is read): unpacking needs no branch
                const size_t src = (size_t)(t0 + pt) * HD;
                const uint32_t dm = st + P::F_BYTES + pt * HD, dl = dm + P::N_BYTES;
#pragma unroll
                for (int v = 0; v < ROW_OPS; ++v) {
                    if (code < 2) cp_async16(dm + v * 16, M + src + v * 16);
                    else st_shared_row16(dm + v * 16, 0x88888888u);
                    if (code == 0) cp_async16(dl + v * 16, L + src + v * 16);
                    else st_shared_row16(dl + v * 16, code == 1 ? 0x88888888u : 0u);
                }
            }
        }
    };

    // Reassemble raw stage rslot into ready slot dslot: token rows of D/2 fp16x2 words [lo_e, f_e, lo_o, f_o].
    // Piece = (token, 8 channels): 8 raw bytes in, 16 ready bytes out; consecutive threads take consecutive
    // pieces, so neither side has bank conflicts.
    auto unpack = [&](int rslot, int dslot) {
        const uint32_t raw = base + (uint32_t)rslot * P::RAW_BYTES;
        const uint32_t rdy = base + P::RDY_OFF + (uint32_t)dslot * P::RDY_BYTES;
        const uint32_t ma = base + P::META_OFF + (uint32_t)rslot * P::META_BYTES;
        if (pt < TOK) {
            const uint32_t s2 = lds32(ma + pt * 4);
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(rdy + P::KV_BYTES + pt * 4), "r"(s2) : "memory");
        }
        uint2 f[ITEMS];
        uint32_t lean[ITEMS], m[ITEMS], l[ITEMS];
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int item = k * NS + pt;
            const int t = item / (D / 8);
            f[k] = lds64(raw + item * 8);
            lean[k] = lds32(ma + TOK * 4 + (t >> 5) * 4);     // warp-uniform: a warp's 32 pieces span 2 tokens
        }
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int item = k * NS + pt;
            m[k] = 0x88888888u;
            l[k] = 0u;
            if (!lean[k]) {
                m[k] = lds32(raw + P::F_BYTES + item * 4);
                l[k] = lds32(raw + P::F_BYTES + P::N_BYTES + item * 4);
            }
        }
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int item = k * NS + pt;
            // byte j of le / lo: low byte of the even / odd channel of pair j
            const uint32_t le = (m[k] & 0xF0F0F0F0u) | ((l[k] >> 4) & 0x0F0F0F0Fu);
            const uint32_t lo = ((m[k] << 4) & 0xF0F0F0F0u) | (l[k] & 0x0F0F0F0Fu);
            const uint32_t a0 = __byte_perm(le, lo, 0x5140), a1 = __byte_perm(le, lo, 0x7362);  // [le,lo] x2
            const uint32_t w0 = __byte_perm(a0, f[k].x, 0x5140), w1 = __byte_perm(a0, f[k].x, 0x7362);
            const uint32_t w2 = __byte_perm(a1, f[k].y, 0x5140), w3 = __byte_perm(a1, f[k].y, 0x7362);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(rdy + item * 16), "r"(w0), "r"(w1), "r"(w2),
                         "r"(w3) : "memory");
        }
    };

    for (int j = 0; j < SA && j < nst; ++j) stage_s(j);
    cp_async_commit();
    cp_async_wait<0>();
    bar_sync(1, NS);
    for (int j = 0; j < RAW - 1; ++j) {
        if (j < nst) issue(j, j);
        cp_async_commit();
    }
    int rslot = 0;
    for (int i = 0; i < nst; ++i) {
        cp_async_wait<RAW - 2>();
        bar_sync(1, NS);   // every staging thread's copies of stage i have landed; stage i-1 is fully unpacked
        const int jr = (rslot == 0) ? RAW - 1 : rslot - 1;
        if (i + RAW - 1 < nst) issue(i + RAW - 1, jr);
        cp_async_commit();
        const int dslot = i % RDY;
        if (i >= RDY) bar_sync(3 + 2 * dslot, NT);   // chain warps are done with this ready slot
        if (!(p.debug & 4)) unpack(rslot, dslot);
        __threadfence_block();
        bar_arrive(2 + 2 * dslot, NT);
        rslot = (rslot + 1 == RAW) ? 0 : rslot + 1;
    }
    cp_async_wait<0>();
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

template <int RAW, int RDY, int D, int NSTG>
static int launch_v_fast(const VParams& p, int BH, cudaStream_t st) {
    size_t smem = (size_t)VPlan<D, RAW, RDY>::BYTES;
    cudaError_t e = cudaFuncSetAttribute(v_compute_kernel<RAW, RDY, D, NSTG>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_status(e, "v_cache_compute smem attribute");
    v_compute_kernel<RAW, RDY, D, NSTG><<<BH, D / 2 + 32 * NSTG, smem, st>>>(p);
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
    p.pf_dist = tuning().v_prefetch;
    p.debug = tuning().debug;
    const int BH = bsz * H;
    const bool fast = D == 128 && aligned16(first8) && aligned16(mid4) && aligned16(last4) &&
                      (n == 0 || (aligned16(s) && s_last_dim % 8 == 0)) &&
                      ((reinterpret_cast<uintptr_t>(o) & 3u) == 0);
    if (fast) {
        const int stages = tuning().v_stages;
        if (stages == 4) return launch_v_fast<4, 2, 128, 4>(p, BH, st);
        if (stages == 8) return launch_v_fast<3, 2, 128, 8>(p, BH, st);
        return launch_v_fast<4, 2, 128, 8>(p, BH, st);
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
