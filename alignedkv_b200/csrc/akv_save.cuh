// Device-side bodies of the plane writers, shared by the stand-alone writer kernels (akv_save.cu) and the fused
// append + flush kernel of the decode step (akv_decode.cu).
#pragma once
#include "akv_common.cuh"

namespace akv {

// 8 channels of one V token (four words [lo_even, hi_even, lo_odd, hi_odd]) -> 8 high bytes, 4 mid bytes, 4 low bytes
// (extension/csrc/V_cache.cu:30-39: adjacent channels share a nibble byte, even channel in the high nibble).
__device__ __forceinline__ void v_split4(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3,  // 8 channels
                                         uint32_t& hi01, uint32_t& hi23, uint32_t& mid, uint32_t& last) {
    hi01 = __byte_perm(w0, w1, 0x7531);
    hi23 = __byte_perm(w2, w3, 0x7531);
    uint32_t x01 = __byte_perm(w0, w1, 0x6420);  // [lo_e0, lo_o0, lo_e1, lo_o1]
    uint32_t x23 = __byte_perm(w2, w3, 0x6420);
    uint32_t m01 = (x01 & 0x00F000F0u) | ((x01 >> 12) & 0x000F000Fu);  // bytes 0 and 2 hold the pair bytes
    uint32_t m23 = (x23 & 0x00F000F0u) | ((x23 >> 12) & 0x000F000Fu);
    uint32_t l01 = ((x01 << 4) & 0x00F000F0u) | ((x01 >> 8) & 0x000F000Fu);
    uint32_t l23 = ((x23 << 4) & 0x00F000F0u) | ((x23 >> 8) & 0x000F000Fu);
    mid = __byte_perm(m01, m23, 0x6420);
    last = __byte_perm(l01, l23, 0x6420);
}

// 32 consecutive channels of one V token (a0..a3 = its 64 input bytes): writes 32 + 16 + 16 plane bytes with 16-byte
// stores.
__device__ __forceinline__ void v_write32(uint4 a0, uint4 a1, uint4 a2, uint4 a3, uint8_t* __restrict__ f_dst,
                                          uint8_t* __restrict__ m_dst, uint8_t* __restrict__ l_dst) {
    uint4 f0, f1, m, l;
    v_split4(a0.x, a0.y, a0.z, a0.w, f0.x, f0.y, m.x, l.x);
    v_split4(a1.x, a1.y, a1.z, a1.w, f0.z, f0.w, m.y, l.y);
    v_split4(a2.x, a2.y, a2.z, a2.w, f1.x, f1.y, m.z, l.z);
    v_split4(a3.x, a3.y, a3.z, a3.w, f1.z, f1.w, m.w, l.w);
    reinterpret_cast<uint4*>(f_dst)[0] = f0;
    reinterpret_cast<uint4*>(f_dst)[1] = f1;
    *reinterpret_cast<uint4*>(m_dst) = m;
    *reinterpret_cast<uint4*>(l_dst) = l;
}
// the same, reading the 64 input bytes from GLOBAL memory through the read-only path
__device__ __forceinline__ void v_write32_global(const uint4* __restrict__ src, uint8_t* __restrict__ f_dst,
                                                 uint8_t* __restrict__ m_dst, uint8_t* __restrict__ l_dst) {
    v_write32(__ldg(src), __ldg(src + 1), __ldg(src + 2), __ldg(src + 3), f_dst, m_dst, l_dst);
}

// Stage a [64 tokens][D] fp16 tile in shared memory, token-major; row(t) = global address of token t's D halves.
template <class RowPtr>
__device__ __forceinline__ void stage_tile64(uint8_t* smem, RowPtr row, int D, int tokens = 64) {
    const int pitch = 2 * D;
    const int vec_per_row = pitch >> 4;
    for (int i = threadIdx.x; i < tokens * vec_per_row; i += blockDim.x) {
        int t = i / vec_per_row, v = i - t * vec_per_row;
        *reinterpret_cast<uint4*>(smem + t * pitch + v * 16) = __ldg(reinterpret_cast<const uint4*>(row(t)) + v);
    }
}

// Emit one K block from a staged tile (see k_write_block64).  MAXOUT: also return, per channel, the signed maximum
// over the 64 tokens as fp16 bits in max_out[d] (the prompt's exponent maxima use the signed maximum,
// extension/k_cache_file.py:77-78).
template <bool MAXOUT>
__device__ __forceinline__ void k_emit_block64(const uint8_t* smem, uint8_t* __restrict__ first8,
                                               uint8_t* __restrict__ mid4, uint8_t* __restrict__ last4, long long tile,
                                               int D, uint16_t* max_out) {
    constexpr int DB = 64;
    const int pitch = 2 * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        // the nibble rows this thread adds onto: requested before the gather so that their latency overlaps it
        uint4* mdst = reinterpret_cast<uint4*>(mid4 + (tile * D + d) * (DB / 2));
        uint4* ldst = reinterpret_cast<uint4*>(last4 + (tile * D + d) * (DB / 2));
        uint4 om[2] = {mdst[0], mdst[1]}, ol[2] = {ldst[0], ldst[1]};
        uint32_t f[16], m[8], l[8];
        float mx = -INFINITY;
#pragma unroll
        for (int g = 0; g < 8; ++g) {  // 8 tokens per group
            uint32_t hi[8], lo[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t x = *reinterpret_cast<const uint16_t*>(smem + (g * 8 + j) * pitch + 2 * d);
                if (MAXOUT) mx = fmaxf(mx, __half2float(__ushort_as_half((unsigned short)x)));
                hi[j] = x >> 8;
                lo[j] = x & 0xFFu;
            }
            f[2 * g] = hi[0] | (hi[1] << 8) | (hi[2] << 16) | (hi[3] << 24);
            f[2 * g + 1] = hi[4] | (hi[5] << 8) | (hi[6] << 16) | (hi[7] << 24);
            uint32_t mw = 0, lw = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // token pair (2j, 2j+1) -> one byte, even token in the high nibble
                uint32_t e = lo[2 * j], o = lo[2 * j + 1];
                mw |= ((e & 0xF0u) | (o >> 4)) << (8 * j);
                lw |= (((e & 0x0Fu) << 4) | (o & 0x0Fu)) << (8 * j);
            }
            m[g] = mw;
            l[g] = lw;
        }
        if (MAXOUT) max_out[d] = __half_as_ushort(__float2half_rn(mx));
        uint4* fdst = reinterpret_cast<uint4*>(first8 + (tile * D + d) * DB);
#pragma unroll
        for (int v = 0; v < 4; ++v) fdst[v] = make_uint4(f[4 * v], f[4 * v + 1], f[4 * v + 2], f[4 * v + 3]);
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            om[v].x = __vadd4(om[v].x, m[4 * v]);
            om[v].y = __vadd4(om[v].y, m[4 * v + 1]);
            om[v].z = __vadd4(om[v].z, m[4 * v + 2]);
            om[v].w = __vadd4(om[v].w, m[4 * v + 3]);
            ol[v].x = __vadd4(ol[v].x, l[4 * v]);
            ol[v].y = __vadd4(ol[v].y, l[4 * v + 1]);
            ol[v].z = __vadd4(ol[v].z, l[4 * v + 2]);
            ol[v].w = __vadd4(ol[v].w, l[4 * v + 3]);
            mdst[v] = om[v];
            ldst[v] = ol[v];
        }
    }
}

// One 64-token K block of one (batch, head): the 64 x D fp16 tile is staged in shared memory token-major (as it
// arrives; row(t) gives the global address of token t's D halves), then thread d gathers channel d of all 64
// tokens and emits one 64-byte first_8 row and one 32-byte row of each nibble plane with 16-byte accesses.  Nibble
// rows are read-add-written (bytewise, mod 256) so that the result equals the reference's `+=`
// (extension/csrc/K_cache.cu:49-56) on any prior plane contents.  `tile` = plane tile index (b*H + h)*nmb + block.
template <class RowPtr>
__device__ __forceinline__ void k_write_block64(uint8_t* smem, uint8_t* __restrict__ first8, uint8_t* __restrict__ mid4,
                                                uint8_t* __restrict__ last4, RowPtr row, long long tile, int D) {
    stage_tile64(smem, row, D);
    __syncthreads();
    k_emit_block64<false>(smem, first8, mid4, last4, tile, D, nullptr);
}

}  // namespace akv
