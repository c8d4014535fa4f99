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
};

// stage layout: [F: 64*D][M: 64*D/2][L: 64*D/2][s2: 64 x u32][code: 64 x u8 (+pad to 16)]
__host__ __device__ inline int v_stage_bytes(int D) { return vc::TOK * D * 2 + vc::TOK * 4 + vc::TOK; }

template <int STAGES, int D>
__global__ void __launch_bounds__(D / 2) v_compute_kernel(const VParams p) {
    using namespace vc;
    constexpr int NT = D / 2;               // threads
    constexpr int HD = D / 2;               // nibble row bytes
    constexpr int F_BYTES = TOK * D;
    constexpr int N_BYTES = TOK * HD;
    constexpr int STAGE = F_BYTES + 2 * N_BYTES + TOK * 4 + TOK;
    constexpr int F_OPS = F_BYTES / 16 / NT;   // 16-byte copies per thread for the high-byte plane
    constexpr int ROW_OPS = HD / 16;           // 16-byte copies per nibble row
    static_assert(NT == TOK, "one thread per staged token is required");
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const long long bh = blockIdx.x;
    const int n = p.n;
    const int nst = (n + TOK - 1) / TOK;
    const uint32_t base = smem_u32(smem);
    const uint8_t* F = p.first8 + (size_t)bh * p.max_seq_len * D;
    const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * HD;
    const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * HD;
    const uint16_t* s_row = p.s + (size_t)bh * p.s_last_dim;
    const uint32_t A = ((uint32_t)p.amin[bh] << 10) & 0xFFFFu;

    // probability of the token this thread stages next (token tid of a stage); tokens >= n behave as p = 0
    uint32_t s_next = 0;
    if (tid < TOK && tid < n) s_next = __ldg(s_row + tid);

    auto issue = [&](int j) {
        const uint32_t st = base + (uint32_t)(j % STAGES) * STAGE;
        const int t0 = j * TOK;
        const int cnt = (n - t0) < TOK ? (n - t0) : TOK;
        // high-byte plane: cnt*D contiguous bytes
        const int fbytes = cnt * D;
#pragma unroll
        for (int it = 0; it < F_OPS; ++it) {
            const int off = (it * NT + tid) << 4;
            if (off < fbytes) cp_async16(st + off, F + (size_t)t0 * D + off);
        }
        if (tid < TOK) {
            const uint32_t sb = s_next;
            const int tn = t0 + TOK + tid;
            s_next = (tn < n) ? (uint32_t)__ldg(s_row + tn) : 0u;
            // decision from the bit patterns (V_cache.cu:211,250-251): 16-bit wrap-around, signed compare
            const int diff = (int)(int16_t)(uint16_t)(A - sb);
            int code = p.reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
            if (tid >= cnt) code = 2;
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(st + F_BYTES + 2 * N_BYTES + tid * 4),
                         "r"(sb | (sb << 16)) : "memory");
            asm volatile("st.shared.u8 [%0], %1;\n" ::"r"(st + F_BYTES + 2 * N_BYTES + TOK * 4 + tid),
                         "r"(code) : "memory");
            if (code < 2) {
                const size_t src = (size_t)(t0 + tid) * HD;
#pragma unroll
                for (int v = 0; v < ROW_OPS; ++v)
                    cp_async16(st + F_BYTES + tid * HD + v * 16, M + src + v * 16);
                if (code == 0) {
#pragma unroll
                    for (int v = 0; v < ROW_OPS; ++v)
                        cp_async16(st + F_BYTES + N_BYTES + tid * HD + v * 16, L + src + v * 16);
                }
            }
        }
    };

    for (int j = 0; j < STAGES - 1; ++j) {
        if (j < nst) issue(j);
        cp_async_commit();
    }

    uint32_t acc = 0;
    for (int i = 0; i < nst; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (i + STAGES - 1 < nst) issue(i + STAGES - 1);
        cp_async_commit();

        const uint32_t st = base + (uint32_t)(i % STAGES) * STAGE;
        const uint32_t fa = st + tid * 2;
        const uint32_t ma = st + F_BYTES + tid;
        const uint32_t la = ma + N_BYTES;
        const uint32_t sa = st + F_BYTES + 2 * N_BYTES;
        const uint32_t ca = sa + TOK * 4;
        // Tokens past n in the last stage carry code 2 and probability +0; their stale high bytes could be
        // Inf/NaN patterns, so the loop stops at cnt instead of multiplying them by zero.
        const int cnt = (n - i * TOK) < TOK ? (n - i * TOK) : TOK;
        for (int g = 0; g < cnt; g += 8) {
            const uint2 codes = lds64(ca + g);
            if (codes.x == 0x02020202u && codes.y == 0x02020202u && g + 8 <= cnt) {
                const uint4 sA = lds128(sa + g * 4), sB = lds128(sa + g * 4 + 16);
                const uint32_t s2[8] = {sA.x, sA.y, sA.z, sA.w, sB.x, sB.y, sB.z, sB.w};
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const uint32_t f = lds16(fa + (g + u) * D);
                    acc = hfma2_bits(__byte_perm(f, 0x80u, 0x1404), s2[u], acc);  // [0x80, f0, 0x80, f1]
                }
            } else {
                const int end = (g + 8 < cnt) ? g + 8 : cnt;
                for (int t = g; t < end; ++t) {
                    const uint32_t code = lds8(ca + t);
                    const uint32_t s2 = lds32(sa + t * 4);
                    const uint32_t f = lds16(fa + t * D);
                    uint32_t mb = 0x88u, lb = 0x00u;
                    if (code < 2) {
                        mb = lds8(ma + t * HD);
                        lb = (code == 0) ? lds8(la + t * HD) : 0x88u;
                    }
                    // even channel: high nibbles; odd channel: low nibbles
                    const uint32_t lo_e = (mb & 0xF0u) | (lb >> 4);
                    const uint32_t lo_o = ((mb & 0x0Fu) << 4) | (lb & 0x0Fu);
                    const uint32_t lo = lo_e | (lo_o << 8);
                    acc = hfma2_bits(__byte_perm(f, lo, 0x1504), s2, acc);  // [lo_e, f0, lo_o, f1]
                }
            }
        }
    }
    cp_async_wait<0>();
    reinterpret_cast<uint32_t*>(p.o)[(size_t)bh * (D / 2) + tid] = acc;
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

template <int STAGES, int D>
static int launch_v_fast(const VParams& p, int BH, cudaStream_t st) {
    size_t smem = (size_t)STAGES * v_stage_bytes(D);
    cudaError_t e = cudaFuncSetAttribute(v_compute_kernel<STAGES, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return cuda_status(e, "v_cache_compute smem attribute");
    v_compute_kernel<STAGES, D><<<BH, D / 2, smem, st>>>(p);
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
    const int BH = bsz * H;
    const bool fast = D == 128 && aligned16(first8) && aligned16(mid4) && aligned16(last4) &&
                      ((reinterpret_cast<uintptr_t>(o) & 3u) == 0);
    if (fast) return launch_v_fast<6, 128>(p, BH, st);
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
