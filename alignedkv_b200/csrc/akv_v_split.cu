// Order-free P.V: the same plane-skipping rule as the exact kernel (akv_v_compute.cu), but the token axis is split
// across CTAs and products are accumulated in fp32, so the sum no longer follows the reference's token order.
//
// The reference's v_cache_compute_kernel (extension/csrc/V_cache.cu:178-308) accumulates every output channel in
// fp16, token by token; that order leaves only B*Hq chains and cannot fill a GPU when B*Hq is small or the
// sequence is long (one (batch, head) over 131072 tokens is a 131072-step dependent chain).  This variant keeps
// the reference's read decisions and substitute constants bit for bit (V_cache.cu:211,250-253) - the bytes it
// fetches are the same - and differs only in the arithmetic of the sum: fp32 partial sums per token chunk, added in
// chunk order, rounded to fp16 once.  Its result is closer to exact arithmetic than the reference's; against the
// reference kernel it differs by the reference's own fp16 accumulation error.
//
// Kernel 1 (v_split_kernel): grid (chunks, B*Hkv), 4 warps.  A warp takes 32-token tiles of the chunk; lane
//   (r, cg) owns tokens 8r..8r+7 of the tile and channels 16cg..16cg+15: one 16-byte load per token row for the
//   high bytes (eight in flight per lane), 8-byte loads of the mid / low rows only for the tokens whose code asks
//   for them (for grouped-query attention: the union over the group's heads; each head then applies its own code).
// Kernel 2 (v_combine_kernel): adds the chunk partials in chunk order and writes fp16 (and optionally fp32).
// Also here: the log-sum-exp merge of per-rank partial attention results for sequence-sharded caches.
#include "akv_common.cuh"

namespace akv {

struct VSplitParams {
    const uint8_t* first8;
    const uint8_t* mid4;
    const uint8_t* last4;
    const uint16_t* s;      // probabilities, one row per (batch, query head)
    const uint8_t* amin;    // threshold byte per (batch, query head)
    float* partial;         // [B*Hq, chunks, D]
    int max_seq_len, s_last_dim, n, reference, chunk_tokens, chunks;
};

__device__ __forceinline__ uint4 ldg128_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg64_stream(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ float2 h2f2(uint32_t h2) {
    return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}

// acc[0..15] += p * value(channel 16cg + k), values rebuilt from 16 high bytes and the per-channel low bytes
// lo_e (even channels of each pair, 8 bytes) / lo_o (odd channels).
__device__ __forceinline__ void fma16(float (&acc)[16], float pf, const uint4& hi, uint2 lo_e, uint2 lo_o) {
    const uint32_t hw[4] = {hi.x, hi.y, hi.z, hi.w};
    const uint32_t le[2] = {lo_e.x, lo_e.y}, lo[2] = {lo_o.x, lo_o.y};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        // word j holds high bytes of channels 4j..4j+3 = pairs 2j, 2j+1; low bytes of pair q are le[q/4] byte q%4
        const uint32_t lew = le[j >> 1] >> ((j & 1) * 16), low = lo[j >> 1] >> ((j & 1) * 16);
        const uint32_t lob = (lew & 0xFFu) | ((low & 0xFFu) << 8) | ((lew & 0xFF00u) << 8) | ((low & 0xFF00u) << 16);
        // lob bytes: [lo(4j), lo(4j+1), lo(4j+2), lo(4j+3)]
        const float2 a = h2f2(__byte_perm(hw[j], lob, 0x1504));   // [lo0, hi0, lo1, hi1]
        const float2 b = h2f2(__byte_perm(hw[j], lob, 0x3726));   // [lo2, hi2, lo3, hi3]
        acc[4 * j + 0] = fmaf(pf, a.x, acc[4 * j + 0]);
        acc[4 * j + 1] = fmaf(pf, a.y, acc[4 * j + 1]);
        acc[4 * j + 2] = fmaf(pf, b.x, acc[4 * j + 2]);
        acc[4 * j + 3] = fmaf(pf, b.y, acc[4 * j + 3]);
    }
}

template <int G>
__global__ void __launch_bounds__(128) v_split_kernel(const VSplitParams p) {
    constexpr int D = 128, HD = 64;
    __shared__ float red[3][G][D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 3, cg = lane & 7;
    const long long bh = blockIdx.y;
    const int chunk = blockIdx.x;
    const int c0 = chunk * p.chunk_tokens;
    const int c1 = min(p.n, c0 + p.chunk_tokens);
    const uint8_t* F = p.first8 + (size_t)bh * p.max_seq_len * D + cg * 16;
    const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * HD + cg * 8;
    const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * HD + cg * 8;
    const uint16_t* s_rows = p.s + (size_t)bh * G * p.s_last_dim;
    uint32_t A[G];
#pragma unroll
    for (int g = 0; g < G; ++g) A[g] = ((uint32_t)p.amin[bh * G + g] << 10) & 0xFFFFu;
    float acc[G][16];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int k = 0; k < 16; ++k) acc[g][k] = 0.f;

    for (int tile0 = c0 + warp * 32; tile0 < c1; tile0 += 4 * 32) {
        const int t0 = tile0 + 8 * r;                 // this lane's 8 tokens: t0 .. t0+7
        // probabilities of the 8 tokens for every head of the group (rows are padded: s_last_dim % 8 == 0)
        uint4 pw[G];
#pragma unroll
        for (int g = 0; g < G; ++g)
            pw[g] = (t0 < c1) ? *reinterpret_cast<const uint4*>(s_rows + (size_t)g * p.s_last_dim + t0)
                              : make_uint4(0, 0, 0, 0);
        uint4 hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            hi[i] = (t0 + i < c1) ? ldg128_stream(F + (size_t)(t0 + i) * D) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (t0 + i >= c1) break;
            uint32_t sb[G];
            int code[G];
            int ucode = 2;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const uint32_t w = (i >> 1) == 0 ? pw[g].x : (i >> 1) == 1 ? pw[g].y : (i >> 1) == 2 ? pw[g].z : pw[g].w;
                sb[g] = (i & 1) ? (w >> 16) : (w & 0xFFFFu);
                const int diff = (int)(int16_t)(uint16_t)(A[g] - sb[g]);
                code[g] = p.reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
                ucode = code[g] < ucode ? code[g] : ucode;
            }
            if (ucode == 2) {
                // no head reads a nibble plane of this token: low bytes 0x80 for every channel
                const uint2 c80 = make_uint2(0x80808080u, 0x80808080u);
#pragma unroll
                for (int g = 0; g < G; ++g)
                    fma16(acc[g], __half2float(__ushort_as_half((unsigned short)sb[g])), hi[i], c80, c80);
            } else {
                const uint2 mrow = ldg64_stream(M + (size_t)(t0 + i) * HD);
                const uint2 lrow = (ucode == 0) ? ldg64_stream(L + (size_t)(t0 + i) * HD) : make_uint2(0, 0);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    // the head's own code picks the bytes or the reference's substitutes (V_cache.cu:250-253)
                    uint2 mb = mrow, lb = lrow;
                    if (code[g] == 2) { mb = make_uint2(0x88888888u, 0x88888888u); lb = make_uint2(0, 0); }
                    else if (code[g] == 1) lb = make_uint2(0x88888888u, 0x88888888u);
                    uint2 lo_e, lo_o;
                    lo_e.x = (mb.x & 0xF0F0F0F0u) | ((lb.x >> 4) & 0x0F0F0F0Fu);
                    lo_e.y = (mb.y & 0xF0F0F0F0u) | ((lb.y >> 4) & 0x0F0F0F0Fu);
                    lo_o.x = ((mb.x << 4) & 0xF0F0F0F0u) | (lb.x & 0x0F0F0F0Fu);
                    lo_o.y = ((mb.y << 4) & 0xF0F0F0F0u) | (lb.y & 0x0F0F0F0Fu);
                    fma16(acc[g], __half2float(__ushort_as_half((unsigned short)sb[g])), hi[i], lo_e, lo_o);
                }
            }
        }
    }
    // sum over the 4 token groups of the warp, then over the 4 warps
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float v = acc[g][k];
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
            acc[g][k] = v;
        }
    if (warp > 0 && r == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int k = 0; k < 16; ++k) red[warp - 1][g][cg * 16 + k] = acc[g][k];
    }
    __syncthreads();
    if (warp == 0 && r == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float* dst = p.partial + (((size_t)bh * G + g) * p.chunks + chunk) * D + cg * 16;
#pragma unroll
            for (int k = 0; k < 16; ++k)
                dst[k] = ((acc[g][k] + red[0][g][cg * 16 + k]) + red[1][g][cg * 16 + k]) + red[2][g][cg * 16 + k];
        }
    }
}

// out[bhq, d] = sum over chunks (in chunk order) of partial[bhq, chunk, d]; fp16 and / or fp32 outputs.
__global__ void __launch_bounds__(128)
v_combine_kernel(const float* __restrict__ partial, __half* __restrict__ o16, float* __restrict__ o32, int chunks, int D) {
    const long long bhq = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = 0.f;
        for (int c = 0; c < chunks; ++c) v += partial[((size_t)bhq * chunks + c) * D + d];
        if (o16) o16[(size_t)bhq * D + d] = __float2half_rn(v);
        if (o32) o32[(size_t)bhq * D + d] = v;
    }
}

// Chunking of the token axis: enough CTAs to fill the GPU several times over, chunks a multiple of 128 tokens.
static void split_plan(int BH, int n, int* chunk_tokens, int* chunks) {
    const int target = sm_count() * 8;
    int want = (target + BH - 1) / BH;
    if (want < 1) want = 1;
    int ct = (n + want - 1) / want;
    ct = ((ct + 127) / 128) * 128;
    if (ct < 256) ct = 256;
    *chunk_tokens = ct;
    *chunks = n > 0 ? (n + ct - 1) / ct : 1;
}

// The streaming form (akv_v_stream.cuh; multi-head attention, aligned mode) wants about three long-lived CTAs per SM:
// fewer, longer chunks than the direct form - so the direct form's plan bounds the scratch of both.
static void stream_plan(int BH, int n, int* chunk_tokens, int* chunks) {
    const int per_sm = tuning().v_split_cps > 0 ? tuning().v_split_cps : 3;
    const int target = sm_count() * per_sm;
    int want = (target + BH - 1) / BH;
    if (want < 1) want = 1;
    int ct = (n + want - 1) / want;
    ct = ((ct + 127) / 128) * 128;
    if (ct < 512) ct = 512;
    *chunk_tokens = ct;
    *chunks = n > 0 ? (n + ct - 1) / ct : 1;
}
int launch_v_split_stream(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*, const uint8_t*,
                          const uint8_t*, int, float*, int, int, int, int, int, int, cudaStream_t);

// true when launch_v_split_probe runs the streaming form, which can compute the threshold bytes itself
bool v_split_takes_probe(int group, int reference, int n) {
    return group == 1 && !reference && tuning().v_split_impl == 0 && n >= 512;
}

long long v_split_scratch_bytes(int bsz, int H, int group, int n) {
    int ct, ch;
    split_plan(bsz * H, n, &ct, &ch);
    return (long long)bsz * H * group * ch * 128 * (long long)sizeof(float);
}

// Order-free P.V over n quantized tokens (head_dim 128).  o16 / o32: [B, Hq, D], either may be null.
// test_o != nullptr (only when v_split_takes_probe() holds): the threshold bytes are computed in the kernel from the
// probe result and the exponent maxima v_exp and written to amin; otherwise they are read from amin.
// o16 == o32 == nullptr: the chunk partials are left in `scratch` for the caller to add up, in chunk order
// (*chunks_out of them per (batch, query head), D floats each).
int launch_v_split_probe(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                         uint8_t* amin, const uint8_t* test_o, const uint8_t* v_exp, uint8_t* o16, float* o32,
                         float* scratch, int* chunks_out, int bsz, int H, int group, int max_seq_len, int D,
                         int s_last_dim, int n, int reference, cudaStream_t st) {
    AKV_REQUIRE(D == 128, AKV_ERR_SHAPE, "v_cache_compute (order-free): head_dim %d is not supported (128 only)", D);
    AKV_REQUIRE(group == 1 || group == 2 || group == 4 || group == 8, AKV_ERR_SHAPE,
                "v_cache_compute (order-free): group size %d is not supported (1, 2, 4, 8)", group);
    AKV_REQUIRE(aligned16(first8) && (reinterpret_cast<uintptr_t>(mid4) & 7u) == 0 &&
                (reinterpret_cast<uintptr_t>(last4) & 7u) == 0 && aligned16(s) && s_last_dim % 8 == 0 &&
                aligned16(scratch), AKV_ERR_ALIGN, "v_cache_compute (order-free): misaligned pointer or row stride");
    AKV_REQUIRE(!test_o || v_split_takes_probe(group, reference, n), AKV_ERR_SHAPE,
                "v_cache_compute (order-free): the probe form needs the streaming kernel");
    const bool combine = o16 != nullptr || o32 != nullptr;
    VSplitParams p;
    p.first8 = first8; p.mid4 = mid4; p.last4 = last4;
    p.s = reinterpret_cast<const uint16_t*>(s);
    p.amin = amin;
    p.partial = scratch;
    p.max_seq_len = max_seq_len; p.s_last_dim = s_last_dim; p.n = n; p.reference = reference;
    int rc;
    if (group == 1 && !reference && tuning().v_split_impl == 0 && n >= 512) {
        stream_plan(bsz * H, n, &p.chunk_tokens, &p.chunks);
        if (chunks_out) *chunks_out = p.chunks;
        rc = launch_v_split_stream(first8, mid4, last4, s, amin, test_o, v_exp, H, scratch, bsz * H, max_seq_len,
                                   s_last_dim, n, p.chunk_tokens, p.chunks, st);
        if (rc != AKV_OK || !combine) return rc;
        count_launch();   // the combine
        v_combine_kernel<<<bsz * H * group, 128, 0, st>>>(scratch, reinterpret_cast<__half*>(o16), o32, p.chunks, D);
        return cuda_status(cudaGetLastError(), "v_cache_compute (order-free) combine launch");
    }
    split_plan(bsz * H, n, &p.chunk_tokens, &p.chunks);
    if (chunks_out) *chunks_out = p.chunks;
    dim3 grid(p.chunks, bsz * H);
    count_launch(combine ? 2 : 1);   // the split pass and the combine
    if (group == 1) v_split_kernel<1><<<grid, 128, 0, st>>>(p);
    else if (group == 2) v_split_kernel<2><<<grid, 128, 0, st>>>(p);
    else if (group == 4) v_split_kernel<4><<<grid, 128, 0, st>>>(p);
    else v_split_kernel<8><<<grid, 128, 0, st>>>(p);
    rc = cuda_status(cudaGetLastError(), "v_cache_compute (order-free) launch");
    if (rc != AKV_OK || !combine) return rc;
    v_combine_kernel<<<bsz * H * group, 128, 0, st>>>(scratch, reinterpret_cast<__half*>(o16), o32, p.chunks, D);
    return cuda_status(cudaGetLastError(), "v_cache_compute (order-free) combine launch");
}

int launch_v_split(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* s,
                   const uint8_t* amin, uint8_t* o16, float* o32, float* scratch, int bsz, int H, int group,
                   int max_seq_len, int D, int s_last_dim, int n, int reference, cudaStream_t st) {
    return launch_v_split_probe(first8, mid4, last4, s, const_cast<uint8_t*>(amin), nullptr, nullptr, o16, o32, scratch,
                                nullptr, bsz, H, group, max_seq_len, D, s_last_dim, n, reference, st);
}

// ------------------------------------------------------------------ log-sum-exp merge of per-rank partial results
// Rank g of R holds, per (batch, head) row i: m[g,i] (maximum score of its tokens), l[g,i] (sum of exp(score - m)),
// o[g,i,:] (attention output over its tokens, normalised by l).  The merged output is
//   out[i,:] = sum_g w_g o[g,i,:],  w_g = l_g exp(m_g - M) / sum_g' l_g' exp(m_g' - M),  M = max_g m_g.
// Input rows are packed as the ranks exchange them: [R, rows, D + 2] fp32 = (m, l, o[0..D-1]).
__global__ void __launch_bounds__(128)
lse_merge_kernel(const float* __restrict__ packed, __half* __restrict__ out, int R, int rows, int D) {
    const int i = blockIdx.x;
    const int W = D + 2;
    lse_merge_row([&](int g, int c) { return packed[((size_t)g * rows + i) * W + c]; }, R, D, out + (size_t)i * D,
                  threadIdx.x, blockDim.x);
}

int launch_lse_merge(const float* packed, uint8_t* out, int R, int rows, int D, cudaStream_t st) {
    count_launch();
    lse_merge_kernel<<<rows, 128, 0, st>>>(packed, reinterpret_cast<__half*>(out), R, rows, D);
    return cuda_status(cudaGetLastError(), "lse_merge launch");
}

}  // namespace akv
