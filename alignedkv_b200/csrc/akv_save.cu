// Plane writers: split fp16 K / V tokens into the high-byte, mid-nibble and low-nibble planes.
//
// Replaces the reference's k_cache_save_prefill_kernel / k_cache_save_decoding_kernel
// (extension/csrc/K_cache.cu:19-94) and v_cache_save_kernel (extension/csrc/V_cache.cu:17-41) with writers that
// produce the same bytes using 128-bit loads and stores wherever the layout allows it.
#include "akv_common.cuh"

namespace akv {

// ================================================================== V
// One thread turns 32 consecutive channels of one token (64 input bytes) into 32 high bytes, 16 mid bytes and
// 16 low bytes: two 16-byte stores into first_8, one each into mid_4 and last_4.

__device__ __forceinline__ void v_split4(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3,  // 8 channels
                                         uint32_t& hi01, uint32_t& hi23, uint32_t& mid, uint32_t& last) {
    // word = [lo_even, hi_even, lo_odd, hi_odd]
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

__global__ void __launch_bounds__(256)
v_save_vec_kernel(uint8_t* __restrict__ first8, uint8_t* __restrict__ mid4, uint8_t* __restrict__ last4,
                  const uint8_t* __restrict__ v_new, int H, int max_seq_len, int D, int start_pos, int seq_len,
                  int v_new_tokens, long long total) {
    const int per_tok = D >> 5;  // threads per token row
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int c = (int)(i % per_tok);
        long long r = i / per_tok;
        int p = (int)(r % seq_len);
        long long bh = r / seq_len;
        int h = (int)(bh % H);
        long long b = bh / H;
        const uint4* src = reinterpret_cast<const uint4*>(
            v_new + 2 * (((b * v_new_tokens + p) * H + h) * (long long)D + c * 32));
        uint4 a0 = __ldg(src), a1 = __ldg(src + 1), a2 = __ldg(src + 2), a3 = __ldg(src + 3);
        uint4 f0, f1, m, l;
        v_split4(a0.x, a0.y, a0.z, a0.w, f0.x, f0.y, m.x, l.x);
        v_split4(a1.x, a1.y, a1.z, a1.w, f0.z, f0.w, m.y, l.y);
        v_split4(a2.x, a2.y, a2.z, a2.w, f1.x, f1.y, m.z, l.z);
        v_split4(a3.x, a3.y, a3.z, a3.w, f1.z, f1.w, m.w, l.w);
        long long row = (bh * max_seq_len + (start_pos + p));
        uint4* fdst = reinterpret_cast<uint4*>(first8 + row * D + c * 32);
        fdst[0] = f0;
        fdst[1] = f1;
        *reinterpret_cast<uint4*>(mid4 + row * (D >> 1) + c * 16) = m;
        *reinterpret_cast<uint4*>(last4 + row * (D >> 1) + c * 16) = l;
    }
}

// Any even head_dim: one thread per channel pair.
__global__ void __launch_bounds__(256)
v_save_pair_kernel(uint8_t* __restrict__ first8, uint8_t* __restrict__ mid4, uint8_t* __restrict__ last4,
                   const uint8_t* __restrict__ v_new, int H, int max_seq_len, int D, int start_pos, int seq_len,
                   int v_new_tokens, long long total) {
    const int hd = D >> 1;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int c = (int)(i % hd);
        long long r = i / hd;
        int p = (int)(r % seq_len);
        long long bh = r / seq_len;
        int h = (int)(bh % H);
        long long b = bh / H;
        uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(
            v_new + 2 * (((b * v_new_tokens + p) * H + h) * (long long)D + 2 * c)));
        long long row = (bh * max_seq_len + (start_pos + p));
        *reinterpret_cast<uint16_t*>(first8 + row * D + 2 * c) = (uint16_t)__byte_perm(w, 0, 0x4431);
        mid4[row * hd + c] = (uint8_t)((w & 0xF0u) | ((w >> 20) & 0x0Fu));
        last4[row * hd + c] = (uint8_t)(((w << 4) & 0xF0u) | ((w >> 16) & 0x0Fu));
    }
}

int launch_v_save(uint8_t* first8, uint8_t* mid4, uint8_t* last4, const uint8_t* v_new, int bsz, int H,
                  int max_seq_len, int D, int start_pos, int seq_len, int v_new_tokens, cudaStream_t st) {
    const bool vec = (D % 32 == 0) && aligned16(first8) && aligned16(mid4) && aligned16(last4) && aligned16(v_new);
    long long total = (long long)bsz * H * seq_len * (vec ? (D >> 5) : (D >> 1));
    long long want = (total + 255) / 256;
    int grid = (int)(want < (long long)sm_count() * 8 ? want : (long long)sm_count() * 8);
    if (grid < 1) grid = 1;
    if (vec)
        v_save_vec_kernel<<<grid, 256, 0, st>>>(first8, mid4, last4, v_new, H, max_seq_len, D, start_pos, seq_len,
                                                v_new_tokens, total);
    else
        v_save_pair_kernel<<<grid, 256, 0, st>>>(first8, mid4, last4, v_new, H, max_seq_len, D, start_pos,
                                                 seq_len, v_new_tokens, total);
    return cuda_status(cudaGetLastError(), "v_cache_save launch");
}

// ================================================================== K
// Block writer, 64-token blocks: one CTA per (batch, head, block).  The 64 x D fp16 tile is staged in shared
// memory token-major (as it arrives), then thread d gathers channel d of all 64 tokens and emits one 64-byte
// first_8 row and one 32-byte row of each nibble plane with 16-byte accesses.  Nibble rows are read-add-written
// (bytewise, mod 256) so that the result equals the reference's `+=` on any prior plane contents.

template <int DB>  // DB = 64
__global__ void __launch_bounds__(256)
k_save_block64_kernel(uint8_t* __restrict__ first8, uint8_t* __restrict__ mid4, uint8_t* __restrict__ last4,
                      const uint8_t* __restrict__ k_new, int H, int n_max_blocks, int D, int blk0, int seqlen) {
    extern __shared__ __align__(16) uint8_t smem[];  // [64][D] halves, row pitch 2*D bytes
    const int z = blockIdx.x, h = blockIdx.y;
    const long long b = blockIdx.z;
    const int pitch = 2 * D;
    // stage: 64 rows of 2*D bytes, 16 bytes per access
    const int vec_per_row = pitch >> 4;
    for (int i = threadIdx.x; i < DB * vec_per_row; i += blockDim.x) {
        int t = i / vec_per_row, v = i - t * vec_per_row;
        const uint4* src = reinterpret_cast<const uint4*>(
            k_new + 2 * (((b * seqlen + (long long)z * DB + t) * H + h) * (long long)D) + v * 16);
        *reinterpret_cast<uint4*>(smem + t * pitch + v * 16) = __ldg(src);
    }
    __syncthreads();
    const long long tile = ((b * H + h) * n_max_blocks + (z + blk0));
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        uint32_t f[16], m[8], l[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {  // 8 tokens per group
            uint32_t hi[8], lo[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t x = *reinterpret_cast<const uint16_t*>(smem + (g * 8 + j) * pitch + 2 * d);
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
        uint4* fdst = reinterpret_cast<uint4*>(first8 + (tile * D + d) * DB);
#pragma unroll
        for (int v = 0; v < 4; ++v) fdst[v] = make_uint4(f[4 * v], f[4 * v + 1], f[4 * v + 2], f[4 * v + 3]);
        uint4* mdst = reinterpret_cast<uint4*>(mid4 + (tile * D + d) * (DB / 2));
        uint4* ldst = reinterpret_cast<uint4*>(last4 + (tile * D + d) * (DB / 2));
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            uint4 om = mdst[v], ol = ldst[v];
            om.x = __vadd4(om.x, m[4 * v]);
            om.y = __vadd4(om.y, m[4 * v + 1]);
            om.z = __vadd4(om.z, m[4 * v + 2]);
            om.w = __vadd4(om.w, m[4 * v + 3]);
            ol.x = __vadd4(ol.x, l[4 * v]);
            ol.y = __vadd4(ol.y, l[4 * v + 1]);
            ol.z = __vadd4(ol.z, l[4 * v + 2]);
            ol.w = __vadd4(ol.w, l[4 * v + 3]);
            mdst[v] = om;
            ldst[v] = ol;
        }
    }
}

// Any block length / partial blocks: one thread per (batch, head, block, channel) row, tokens in order.
__global__ void __launch_bounds__(128)
k_save_rows_kernel(uint8_t* __restrict__ first8, uint8_t* __restrict__ mid4, uint8_t* __restrict__ last4,
                   const uint8_t* __restrict__ k_new, int H, int n_blocks, int n_max_blocks, int D, int d_block,
                   int blk0, int seqlen, long long total) {
    const int hb = d_block >> 1;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int d = (int)(i % D);
        long long r = i / D;
        int z = (int)(r % n_blocks);
        long long bh = r / n_blocks;
        int h = (int)(bh % H);
        long long b = bh / H;
        int t_lo = z * d_block;
        int t_hi = t_lo + d_block < seqlen ? t_lo + d_block : seqlen;
        long long row = ((bh * n_max_blocks + (z + blk0)) * D + d) * hb;
        for (int t = t_lo; t < t_hi; ++t) {
            int slot = t - t_lo;
            const uint8_t* x = k_new + 2 * (((b * seqlen + t) * H + h) * (long long)D + d);
            uint32_t lo = x[0];
            int sh = (slot & 1) << 2;
            first8[2 * row + slot] = x[1];
            mid4[row + (slot >> 1)] += (uint8_t)((lo & 0xF0u) >> sh);
            last4[row + (slot >> 1)] += (uint8_t)((lo & 0x0Fu) << (4 - sh));
        }
    }
}

// Single token into an existing block (the reference's decoding writer): one thread per (batch, head, channel).
__global__ void __launch_bounds__(128)
k_save_token_kernel(uint8_t* __restrict__ first8, uint8_t* __restrict__ mid4, uint8_t* __restrict__ last4,
                    const uint8_t* __restrict__ k_new, int H, int n_max_blocks, int D, int d_block, int blk,
                    int slot, long long total) {
    const int hb = d_block >> 1;
    const int sh = (slot & 1) << 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int d = (int)(i % D);
        long long bh = i / D;
        long long row = ((bh * n_max_blocks + blk) * D + d) * hb;
        const uint8_t* x = k_new + 2 * (bh * (long long)D + d);  // k_new is [B,1,H,D]
        uint32_t lo = x[0];
        first8[2 * row + slot] = x[1];
        mid4[row + (slot >> 1)] += (uint8_t)((lo & 0xF0u) >> sh);
        last4[row + (slot >> 1)] += (uint8_t)((lo & 0x0Fu) << (4 - sh));
    }
}

int launch_k_save(uint8_t* first8, uint8_t* mid4, uint8_t* last4, const uint8_t* k_new, int bsz, int H,
                  int n_blocks, int n_max_blocks, int D, int d_block, int start_pos, int seqlen, cudaStream_t st) {
    if (start_pos == 0 || seqlen % d_block == 0) {
        if (n_blocks == 0) return AKV_OK;
        const int blk0 = start_pos / d_block;
        const bool full = (long long)n_blocks * d_block <= (long long)seqlen;
        const bool fast = full && d_block == 64 && (D % 8 == 0) && 128 * D <= 96 * 1024 && n_blocks <= 2147483647 &&
                          H <= 65535 && bsz <= 65535 && aligned16(first8) && aligned16(mid4) && aligned16(last4) &&
                          aligned16(k_new);
        if (fast) {
            size_t smem = (size_t)64 * 2 * D;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(k_save_block64_kernel<64>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return cuda_status(e, "k_cache_save smem attribute");
            }
            dim3 grid(n_blocks, H, bsz);
            int threads = D < 256 ? ((D + 31) / 32) * 32 : 256;
            k_save_block64_kernel<64><<<grid, threads, smem, st>>>(first8, mid4, last4, k_new, H, n_max_blocks, D,
                                                                   blk0, seqlen);
        } else {
            long long total = (long long)bsz * H * n_blocks * D;
            long long want = (total + 127) / 128;
            int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
            k_save_rows_kernel<<<grid, 128, 0, st>>>(first8, mid4, last4, k_new, H, n_blocks, n_max_blocks, D,
                                                     d_block, blk0, seqlen, total);
        }
        return cuda_status(cudaGetLastError(), "k_cache_save launch");
    } else if (seqlen == 1) {
        const int blk = start_pos / d_block;
        const int slot = start_pos - blk * d_block;
        long long total = (long long)bsz * H * D;
        long long want = (total + 127) / 128;
        int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
        k_save_token_kernel<<<grid, 128, 0, st>>>(first8, mid4, last4, k_new, H, n_max_blocks, D, d_block, blk,
                                                  slot, total);
        return cuda_status(cudaGetLastError(), "k_cache_save launch");
    }
    return AKV_OK;  // the reference does nothing for any other (start_pos, seqlen) pair
}

}  // namespace akv
