// Shared device/host helpers of the alignedkv_b200 kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/alignedkv_b200.h"

namespace akv {

// ---------------------------------------------------------------- error plumbing (host)
void set_error(const char* fmt, ...);
int cuda_status(cudaError_t e, const char* what);
int sm_count();          // SMs of the current device (cached per device)
int max_dyn_smem();      // opt-in dynamic shared memory per block of the current device
void count_launch(int n = 1);   // every kernel launch of this library is counted (akv_launch_count)

// Launch-shape knobs (defaults are the measured best on B200); see akv_set_tuning().
struct Tuning {
    int k_kch = 16;     // channels per stage of the q.K^T kernel (8 or 16)
    int k_stages = 3;   // ring depth per warp of the q.K^T kernel (3..6, see launch_k_compute)
    int timing = 0;     // 1: akv_decode_step records CUDA events around its two streaming kernels
    int k_wpc = 0;      // cap on warps per CTA of the q.K^T kernel (0 = as many as shared memory allows)
    int pdl = 1;        // 1: the kernels of a decode step are chained with programmatic dependent launch
    int k_gqa_kch = 8;  // channels per stage of the q.K^T kernel when query heads share KV heads (8 or 16)
    int v_impl = 0;     // exact P.V, multi-head, aligned mode: 0 = branch-free chain form, 1 = producer-transposed form
    int v_nf = 0;       // exact P.V (form 0): cap on the ring depth in 64-token stages (0 = from the shared-memory budget)
    int v_nside = 0;    // exact P.V (form 0): rows of the nibble side ring, a power of two >= 128 (0 = default)
    int v_cps = 0;      // exact P.V (form 0): CTAs per SM the shared-memory budget is cut for (0 = one wave)
    int v_upc = 0;      // exact P.V (form 0): (batch, head) units per CTA, 1 or 2 (0 = default)
    int v_gqa_form = 0;   // exact P.V, grouped queries (form 0): 0 = by size, 1 = one ring per query head, 2 = the group's heads share a ring
    int v_npt = 0;      // exact P.V (form 0): low-byte tables per head, 2, 4, 6 or 8 (0 = default)
    int v_ndw = 0;      // exact P.V (form 0), two rings of one head each: decision warps per head, 2 or 4 (0 = default)
    int v_split_impl = 0;   // order-free P.V, multi-head, aligned mode: 0 = staged through shared memory by bulk copies, 1 = direct loads
    int v_split_nf = 0;     // order-free P.V, streaming form: ring depth 4 or 8 (0 = default 8)
    int v_split_cps = 0;    // order-free P.V, streaming form: CTAs per SM the chunking aims at (0 = default 3)
};
Tuning& tuning();

#define AKV_REQUIRE(cond, code, ...)          \
    do {                                      \
        if (!(cond)) {                        \
            ::akv::set_error(__VA_ARGS__);    \
            return (code);                    \
        }                                     \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------- programmatic dependent launch
// The kernels of one decode step form a chain in one stream.  Launched with the programmatic-serialization
// attribute, a kernel's CTAs may become resident while its predecessor is still running; every such kernel calls
// pdl_enter() first: it lets ITS successor be scheduled early and then blocks until the predecessor grid has
// completed and its memory is visible.  Without the attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
}
template <class Kernel, class... Args>
static inline cudaError_t launch_chained(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                         Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    count_launch();
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// ---------------------------------------------------------------- async copies global -> shared (LDGSTS)
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte copy that bypasses L1 (streamed data is used once).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- shared-memory loads by 32-bit address
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.u32 [%0], {%1,%2};\n" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint32_t u4w(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];\n" : "=r"(v) : "r"(a));
    return v;
}

// fp16x2 fused multiply-add on raw bit patterns (round-to-nearest-even, denormals kept): the reference's
// __hfma2 (K_cache.cu:304, V_cache.cu:304).
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Threshold byte of P.V for flat row i = b*Hq + h of the reference's [B,Hq,Hq,1] tensor, computed by one warp:
// min_d ((exp(test_o[bb, hp, d]) & 0x1E) + 15 - v_exp[bb, he, d]) mod 256 with bb = i / (Hq*Hq), hp = (i / Hq) % Hq,
// he = i % Hq (extension/v_cache_file.py:142,156-160).  The exponent maxima are stored per KV head; query head he
// belongs to KV head he / G (for G > 1 this is the reference's rule applied to the cache with its KV heads repeated
// G times).  Every lane returns the result.
__device__ __forceinline__ uint32_t v_threshold_warp(const uint16_t* __restrict__ test_o,
                                                     const uint8_t* __restrict__ v_exp, long long i, int H, int G,
                                                     int D, int lane) {
    // (row indices fit 32 bits: launchers reject more than 2^30 rows)
    const uint32_t Hq = (uint32_t)(H * G), iu = (uint32_t)i;
    const uint32_t bb = iu / (Hq * Hq), hp = (iu / Hq) % Hq, he = iu % Hq;
    const uint16_t* trow = test_o + (size_t)(bb * Hq + hp) * D;
    const uint8_t* erow = v_exp + (size_t)(bb * H + he / G) * D;
    uint32_t m = 255;
    for (int d0 = 0; d0 < D; d0 += 128) {       // four loads of each row in flight per lane
        uint32_t t[4], x[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int d = d0 + r * 32 + lane;
            t[r] = d < D ? (uint32_t)trow[d] : 0u;
            x[r] = d < D ? (uint32_t)erow[d] : 0u;
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint32_t e = (t[r] >> 10) & 0x1Eu;
            const uint32_t a = (e + 15u - x[r]) & 0xFFu;
            if (d0 + r * 32 + lane < D) m = min(m, a);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = min(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    return m;
}

// Log-sum-exp merge of one (batch, head) row over R shards (used by lse_merge_kernel and by the peer exchange, which
// must agree bit for bit).  ld(g, c) = float c of shard g's record (m, l, o[0..D-1]); out[d] = sum_g w_g o_g[d],
// w_g = l_g exp(m_g - M) / sum_g' l_g' exp(m_g' - M), M = max_g m_g; shards with l = 0 are ignored.
template <class Load>
__device__ __forceinline__ void lse_merge_row(Load ld, int R, int D, __half* out, int tid, int nthreads) {
    float M = -INFINITY;
    for (int g = 0; g < R; ++g) {
        const float l = ld(g, 1);
        if (l > 0.f) M = fmaxf(M, ld(g, 0));
    }
    float denom = 0.f;
    for (int g = 0; g < R; ++g) {
        const float l = ld(g, 1);
        if (l > 0.f) denom += l * expf(ld(g, 0) - M);
    }
    for (int d = tid; d < D; d += nthreads) {
        float v = 0.f;
        for (int g = 0; g < R; ++g) {
            const float l = ld(g, 1);
            if (l > 0.f) v += (l * expf(ld(g, 0) - M) / denom) * ld(g, 2 + d);
        }
        out[d] = __float2half_rn(denom > 0.f ? v : 0.f);
    }
}

}  // namespace akv
