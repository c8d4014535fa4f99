// Plane writers: split fp16 K / V tokens into the high-byte, mid-nibble and low-nibble planes.
//
// Replaces the reference's k_cache_save_prefill_kernel / k_cache_save_decoding_kernel
// (extension/csrc/K_cache.cu:19-94) and v_cache_save_kernel (extension/csrc/V_cache.cu:17-41) with writers that
// produce the same bytes using 128-bit loads and stores wherever the layout allows it.
#include "akv_save.cuh"

namespace akv {

// ================================================================== V
// One thread turns 32 consecutive channels of one token (64 input bytes) into 32 high bytes, 16 mid bytes and
// 16 low bytes: two 16-byte stores into first_8, one each into mid_4 and last_4 (v_write32, akv_save.cuh).

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
        long long row = (bh * max_seq_len + (start_pos + p));
        v_write32_global(src, first8 + row * D + c * 32, mid4 + row * (D >> 1) + c * 16, last4 + row * (D >> 1) + c * 16);
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
    count_launch();
    if (vec)
        v_save_vec_kernel<<<grid, 256, 0, st>>>(first8, mid4, last4, v_new, H, max_seq_len, D, start_pos, seq_len,
                                                v_new_tokens, total);
    else
        v_save_pair_kernel<<<grid, 256, 0, st>>>(first8, mid4, last4, v_new, H, max_seq_len, D, start_pos,
                                                 seq_len, v_new_tokens, total);
    return cuda_status(cudaGetLastError(), "v_cache_save launch");
}

// ================================================================== K
// Block writer, 64-token blocks: one CTA per (batch, head, block); body in akv_save.cuh (k_write_block64).

template <int DB>  // DB = 64
__global__ void __launch_bounds__(256)
k_save_block64_kernel(uint8_t* __restrict__ first8, uint8_t* __restrict__ mid4, uint8_t* __restrict__ last4,
                      const uint8_t* __restrict__ k_new, int H, int n_max_blocks, int D, int blk0, int seqlen) {
    extern __shared__ __align__(16) uint8_t smem[];  // [64][D] halves, row pitch 2*D bytes
    const int z = blockIdx.x, h = blockIdx.y;
    const long long b = blockIdx.z;
    const long long tile = ((b * H + h) * n_max_blocks + (z + blk0));
    auto row = [&](int t) { return k_new + 2 * (((b * seqlen + (long long)z * DB + t) * H + h) * (long long)D); };
    k_write_block64(smem, first8, mid4, last4, row, tile, D);
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
            count_launch();
            k_save_block64_kernel<64><<<grid, threads, smem, st>>>(first8, mid4, last4, k_new, H, n_max_blocks, D,
                                                                   blk0, seqlen);
        } else {
            long long total = (long long)bsz * H * n_blocks * D;
            long long want = (total + 127) / 128;
            int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
            count_launch();
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
        count_launch();
        k_save_token_kernel<<<grid, 128, 0, st>>>(first8, mid4, last4, k_new, H, n_max_blocks, D, d_block, blk,
                                                  slot, total);
        return cuda_status(cudaGetLastError(), "k_cache_save launch");
    }
    return AKV_OK;  // the reference does nothing for any other (start_pos, seqlen) pair
}

}  // namespace akv
