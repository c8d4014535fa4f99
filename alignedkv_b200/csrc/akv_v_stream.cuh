// Order-free P.V, streaming form (multi-head attention, aligned mode): the split pass of akv_v_split.cu with the high
// bytes staged through shared memory by bulk asynchronous copies.
//
// Same contract as v_split_kernel (see akv_v_split.cu): the reference's read decisions and substitute constants
// (extension/csrc/V_cache.cu:211,250-253) bit for bit, fp32 partial sums per token chunk, which v_combine_kernel adds
// in chunk order and rounds to fp16 once.
//
// Design (B200).  The direct form has every warp load a tile and then compute on it, so its loads are exposed.  Here a
// CTA = one (batch, head, token chunk) has a copy warp that streams the chunk's high bytes as 8 KB stages (64 tokens,
// contiguous in the plane) into a ring, one cp.async.bulk per stage, counted on the stage's mbarrier, and four consumer
// warps that take the stages in turn (the ring depth is a multiple of four: a slot always serves the same warp).  A
// consumer lane owns 16 tokens x 16 channels of its stage: one 16-byte shared
// load per token row, low bytes constant 0x80 - the reference's substitute when no nibble plane is read, which is the
// rule.  The few tokens whose probability lies within two binades of the threshold are left out of that loop (their
// probability counts as 0 there); their nibble rows are requested from global memory BEFORE the loop (up to two per
// lane, the usual case; more are fetched late) and their full contribution is added after it, so that the latency
// of those small loads hides behind the stage's arithmetic.  The probabilities of the next stage are loaded a stage
// ahead.  The order of the sum is free, so none of this changes the contract.
// Every wait is bounded; a wait that runs out raises the device error flag and the CTA writes NaN partial sums.
#pragma once
#include "akv_v_chain.cuh"

namespace akv {

struct VStreamParams {
    const uint8_t* first8;
    const uint8_t* mid4;
    const uint8_t* last4;
    const uint16_t* s;      // probabilities, one row per (batch, head)
    const uint8_t* amin;    // threshold byte per (batch, head)
    // test_o != nullptr: every CTA computes its head's threshold byte itself from the probe result [B,H,D] and the
    // exponent maxima [B,H,D] (v_threshold_warp), and chunk 0 stores it to amin_out
    const uint16_t* test_o;
    const uint8_t* v_exp;
    uint8_t* amin_out;
    int H;
    float* partial;         // [B*H, chunks, D]
    int max_seq_len, s_last_dim, n, chunk_tokens, chunks, nf;
};

namespace vst {
constexpr int TOK = 64, D = 128, HD = 64, F_BYTES = TOK * D, CONSUMERS = 4;
__host__ __device__ inline int smem_bytes(int nf) { return nf * F_BYTES + 2 * nf * 8 + 3 * D * 4; }
}  // namespace vst

__device__ __forceinline__ uint2 vst_ldg64(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ float2 vst_h2f2(uint32_t h2) {
    return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}
// acc[0..15] += p * value(channel 16cg + k): 16 high bytes, low bytes of the even / odd channel of each pair
__device__ __forceinline__ void vst_fma16(float (&acc)[16], float pf, const uint4& hi, uint2 lo_e, uint2 lo_o) {
    const uint32_t hw[4] = {hi.x, hi.y, hi.z, hi.w};
    const uint32_t le[2] = {lo_e.x, lo_e.y}, lo[2] = {lo_o.x, lo_o.y};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t lew = le[j >> 1] >> ((j & 1) * 16), low = lo[j >> 1] >> ((j & 1) * 16);
        const uint32_t lob = (lew & 0xFFu) | ((low & 0xFFu) << 8) | ((lew & 0xFF00u) << 8) | ((low & 0xFF00u) << 16);
        const float2 a = vst_h2f2(__byte_perm(hw[j], lob, 0x1504));
        const float2 b = vst_h2f2(__byte_perm(hw[j], lob, 0x3726));
        acc[4 * j + 0] = fmaf(pf, a.x, acc[4 * j + 0]);
        acc[4 * j + 1] = fmaf(pf, a.y, acc[4 * j + 1]);
        acc[4 * j + 2] = fmaf(pf, b.x, acc[4 * j + 2]);
        acc[4 * j + 3] = fmaf(pf, b.y, acc[4 * j + 3]);
    }
}
// the same with the constant low byte 0x80 on every channel
__device__ __forceinline__ void vst_fma16_lean(float (&acc)[16], float pf, const uint4& hi) {
    const uint32_t hw[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 a = vst_h2f2(__byte_perm(hw[j], 0x80808080u, 0x1404));
        const float2 b = vst_h2f2(__byte_perm(hw[j], 0x80808080u, 0x3424));
        acc[4 * j + 0] = fmaf(pf, a.x, acc[4 * j + 0]);
        acc[4 * j + 1] = fmaf(pf, a.y, acc[4 * j + 1]);
        acc[4 * j + 2] = fmaf(pf, b.x, acc[4 * j + 2]);
        acc[4 * j + 3] = fmaf(pf, b.y, acc[4 * j + 3]);
    }
}

__global__ void __launch_bounds__(160) v_stream_kernel(const VStreamParams p) {
    using namespace vst;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nf = p.nf;
    const long long bh = blockIdx.y;
    const int chunk = blockIdx.x;
    const int c0 = chunk * p.chunk_tokens;
    const int c1 = min(p.n, c0 + p.chunk_tokens);
    const int nst = (c1 - c0 + TOK - 1) / TOK;
    const uint32_t ring = smem_u32(smem);
    const uint32_t bar_full = ring + nf * F_BYTES, bar_free = bar_full + nf * 8;
    float* red = reinterpret_cast<float*>(smem + nf * F_BYTES + 2 * nf * 8);     // [3][D]
    const int r = lane >> 3, cg = lane & 7;                 // consumer lane: token group (16 tokens), channel group (16 channels)
    float acc[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) acc[k] = 0.f;

    pdl_enter();
    {   // the launch must have given the ring its room (uniform over the CTA: all threads leave together)
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;\n" : "=r"(dyn));
        if (nf < CONSUMERS || nf % CONSUMERS != 0 || dyn < (uint32_t)smem_bytes(nf) || (ring & 127u) != 0 || c1 <= c0) {
            if (threadIdx.x == 0) atomicOr(&g_v_wait_gave_up, 2u);
            return;
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < nf; ++s) {
            mbar_init(bar_full + s * 8, 1);    // the copy warp's arrival (+ the stage's bytes)
            mbar_init(bar_free + s * 8, 1);    // the arrival of the consumer warp that took the stage
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    if (warp == CONSUMERS) {
        // ------------------------------------------------------------------ copy warp
        const uint8_t* F = p.first8 + ((size_t)bh * p.max_seq_len + c0) * D;
        int slot = 0;
        uint32_t parity = 0;
        bool alive = true;
#pragma unroll 1
        for (int i = 0; i < nst; ++i) {
            if (i >= nf) {
                alive = mbar_wait(bar_free + slot * 8, parity);
                if (!alive) break;
            }
            if (lane == 0) {
                const int cnt = (c1 - c0 - i * TOK) < TOK ? (c1 - c0 - i * TOK) : TOK;
                mbar_arrive_expect(bar_full + slot * 8, (uint32_t)cnt * D);
                bulk_copy(ring + (uint32_t)slot * F_BYTES, F + (size_t)i * TOK * D, (uint32_t)cnt * D, bar_full + slot * 8);
            }
            if (++slot == nf) { slot = 0; if (i >= nf) parity ^= 1u; }
        }
        if (!alive) v_sleep_ms();
    } else {
        // ------------------------------------------------------------------ consumer warps
        const uint8_t* M = p.mid4 + (size_t)bh * p.max_seq_len * HD + cg * 8;
        const uint8_t* L = p.last4 + (size_t)bh * p.max_seq_len * HD + cg * 8;
        const uint16_t* s_row = p.s + (size_t)bh * p.s_last_dim;
        uint32_t a8;
        if (p.test_o) {
            a8 = v_threshold_warp(p.test_o, p.v_exp, bh, p.H, 1, D, lane);
            if (chunk == 0 && warp == 0 && lane == 0) p.amin_out[bh] = (uint8_t)a8;
        } else {
            a8 = p.amin[bh];
        }
        const uint32_t A = (a8 << 10) & 0xFFFFu;
        const int n8 = (p.n + 7) & ~7;                       // readable extent of the probability row
        bool alive = true;
        // probabilities of this lane's 16 tokens of a stage (two 16-byte loads; the row is padded to 8 values)
        auto load_p = [&](int i, uint4& a, uint4& b) {
            const int t = c0 + i * TOK + r * 16;
            a = (i < nst && t < n8) ? *reinterpret_cast<const uint4*>(s_row + t) : make_uint4(0, 0, 0, 0);
            b = (i < nst && t + 8 < n8) ? *reinterpret_cast<const uint4*>(s_row + t + 8) : make_uint4(0, 0, 0, 0);
        };
        uint4 pa, pb, na, nb;
        load_p(warp, pa, pb);
#pragma unroll 1
        for (int i = warp; i < nst && alive; i += CONSUMERS) {
            load_p(i + CONSUMERS, na, nb);                    // the next stage of this warp
            const int slot = i % nf;
            const uint32_t parity = (uint32_t)(i / nf) & 1u;
            const int tb = c0 + i * TOK + r * 16;             // this lane's first token
            const uint32_t pw[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
            // tokens that read a nibble plane (code < 2): bit t of fm; of those, the ones that read both (code 0): fl
            uint32_t fm = 0, fl = 0;
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                const uint32_t sb = (t & 1) ? (pw[t >> 1] >> 16) : (pw[t >> 1] & 0xFFFFu);
                const int diff = (int)(int16_t)(uint16_t)(A - sb);
                if (tb + t < c1 && diff < 0x0800) fm |= 1u << t;
                if (tb + t < c1 && diff < 0x0400) fl |= 1u << t;
            }
            // the first two flagged tokens of the lane: their nibble rows are requested now and used after the loop
            const int ta = fm ? __ffs(fm) - 1 : -1;
            const uint32_t fm2 = fm & (fm - 1);
            const int tc = fm2 ? __ffs(fm2) - 1 : -1;
            uint2 ma = make_uint2(0, 0), la2 = make_uint2(0x88888888u, 0x88888888u);
            uint2 mc = make_uint2(0, 0), lc = make_uint2(0x88888888u, 0x88888888u);
            if (ta >= 0) {
                ma = vst_ldg64(M + (size_t)(tb + ta) * HD);
                if ((fl >> ta) & 1u) la2 = vst_ldg64(L + (size_t)(tb + ta) * HD);
            }
            if (tc >= 0) {
                mc = vst_ldg64(M + (size_t)(tb + tc) * HD);
                if ((fl >> tc) & 1u) lc = vst_ldg64(L + (size_t)(tb + tc) * HD);
            }
            alive = mbar_wait(bar_full + slot * 8, parity);
            if (!alive) break;
            const uint32_t st = ring + (uint32_t)slot * F_BYTES + (uint32_t)(r * 16) * D + cg * 16;
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                const uint32_t sb = (t & 1) ? (pw[t >> 1] >> 16) : (pw[t >> 1] & 0xFFFFu);
                // (a flagged token counts with probability 0 here; rows beyond the chunk hold stale bytes, which may
                // spell an infinity: they are replaced by zeros, not just weighted with 0)
                const bool in = tb + t < c1;
                const float pf = (in && !((fm >> t) & 1u)) ? __half2float(__ushort_as_half((unsigned short)sb)) : 0.f;
                const uint4 hi = in ? lds128(st + t * D) : make_uint4(0u, 0u, 0u, 0u);
                vst_fma16_lean(acc, pf, hi);
            }
            if (__builtin_expect(fm != 0, 0)) {
                // flagged tokens with their own low bytes (V_cache.cu:250-253); low plane not read: low nibble 8
#pragma unroll 1
                for (uint32_t bits = fm; bits; bits &= bits - 1) {
                    const int t = __ffs(bits) - 1;
                    uint2 mb, lb;
                    if (t == ta) { mb = ma; lb = la2; }
                    else if (t == tc) { mb = mc; lb = lc; }
                    else {
                        mb = vst_ldg64(M + (size_t)(tb + t) * HD);
                        lb = ((fl >> t) & 1u) ? vst_ldg64(L + (size_t)(tb + t) * HD) : make_uint2(0x88888888u, 0x88888888u);
                    }
                    uint2 lo_e, lo_o;
                    lo_e.x = (mb.x & 0xF0F0F0F0u) | ((lb.x >> 4) & 0x0F0F0F0Fu);
                    lo_e.y = (mb.y & 0xF0F0F0F0u) | ((lb.y >> 4) & 0x0F0F0F0Fu);
                    lo_o.x = ((mb.x << 4) & 0xF0F0F0F0u) | (lb.x & 0x0F0F0F0Fu);
                    lo_o.y = ((mb.y << 4) & 0xF0F0F0F0u) | (lb.y & 0x0F0F0F0Fu);
                    const uint32_t w = pw[t >> 1];
                    const uint32_t sb = (t & 1) ? (w >> 16) : (w & 0xFFFFu);
                    const uint4 hi = lds128(st + t * D);
                    vst_fma16(acc, __half2float(__ushort_as_half((unsigned short)sb)), hi, lo_e, lo_o);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_free + slot * 8);
            pa = na; pb = nb;
        }
        // sum over the 4 token groups of the warp
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float v = acc[k];
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
            acc[k] = alive ? v : __int_as_float(0x7FC00000);
        }
        if (warp > 0 && r == 0) {
#pragma unroll
            for (int k = 0; k < 16; ++k) red[(warp - 1) * D + cg * 16 + k] = acc[k];
        }
        if (!alive) v_sleep_ms();
    }
    __syncthreads();
    if (warp == 0 && r == 0) {       // warp 0's sums plus the other three warps', in warp order
        float* dst = p.partial + ((size_t)bh * p.chunks + chunk) * D + cg * 16;
#pragma unroll
        for (int k = 0; k < 16; ++k)
            dst[k] = ((acc[k] + red[cg * 16 + k]) + red[D + cg * 16 + k]) + red[2 * D + cg * 16 + k];
    }
}

// Launches the split pass in its streaming form; chunk_tokens a multiple of 64.
static int launch_v_stream(const VStreamParams& q, int BH, cudaStream_t st) {
    static bool configured[64] = {false};   // the attribute is per device
    VStreamParams p = q;
    // ring depth: a multiple of the consumer warps, so that a ring slot's stages all go to ONE warp, which then sees
    // the slot's barrier phases in order (a parity wait cannot tell phase k from phase k - 2: a warp that asked for
    // stage i + 2 nf's phase before stage i + nf's had completed would be let through)
    p.nf = tuning().v_split_nf == 4 ? 4 : 2 * vst::CONSUMERS;      // (4, 8 and 2..6 CTAs per SM all measure 33-35 us at batch 8 x 32 x 4096)
    const int smem = vst::smem_bytes(p.nf);
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(v_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             vst::smem_bytes(2 * vst::CONSUMERS));     // (the deepest ring in use)
        if (e != cudaSuccess) return cuda_status(e, "v_cache_compute (order-free) smem attribute");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    launch_chained(v_stream_kernel, dim3(p.chunks, BH), dim3(160), (size_t)smem, st, p);
    return cuda_status(cudaGetLastError(), "v_cache_compute (order-free) launch");
}

}  // namespace akv
