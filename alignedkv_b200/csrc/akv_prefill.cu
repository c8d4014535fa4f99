// Prompt ingestion in one pass: what K_Cache_Class.save / V_Cache_Class.save do for start_pos == 0
// (extension/k_cache_file.py:76-96, extension/v_cache_file.py:79-96) - per-channel exponent of the signed maximum over
// the prompt, whole 64-token blocks split into the planes (K1 / V1: extension/csrc/K_cache.cu:19-58,
// extension/csrc/V_cache.cu:17-41), the remaining tokens copied to the fp16 residual buffers - reading every input
// byte once.  The reference makes three passes per tensor (max reduction, plane writer, tail copy).
//
// prefill_kernel: grid (ceil(S/64), H, B), 128 threads.  The CTA stages its 64-token tile of K and of V in shared
// memory (16-byte loads), emits the K block (thread = channel: gathers 64 tokens, 16-byte plane stores) and the V
// rows (thread = 32 channels of a token) and records per channel the signed maximum of the tile; a partial last tile
// goes to the residual buffers instead of the planes.  exp_reduce_kernel then takes the maximum over tiles and stores
// its exponent field.
#include "akv_save.cuh"

namespace akv {

constexpr int PF_BLK = 64;

__global__ void __launch_bounds__(128)
prefill_kernel(uint8_t* __restrict__ k_first_8, uint8_t* __restrict__ k_mid_4, uint8_t* __restrict__ k_last_4,
               uint8_t* __restrict__ v_first_8, uint8_t* __restrict__ v_mid_4, uint8_t* __restrict__ v_last_4,
               uint8_t* __restrict__ restk, uint8_t* __restrict__ restv, const uint8_t* __restrict__ k,
               const uint8_t* __restrict__ v, uint16_t* __restrict__ kmax_part, uint16_t* __restrict__ vmax_part, int H,
               int D, int S, int nmb, int max_seq_len, int tiles) {
    extern __shared__ __align__(16) uint8_t smem[];      // K tile, then V tile: [64][D] halves each
    const int z = blockIdx.x, h = blockIdx.y;
    const long long b = blockIdx.z;
    const long long bh = b * H + h;
    const int t0 = z * PF_BLK;
    const int cnt = min(PF_BLK, S - t0);
    const int pitch = 2 * D;
    uint8_t* ks = smem;
    uint8_t* vs = smem + PF_BLK * pitch;
    auto krow = [&](int t) { return k + 2 * (((b * S + t0 + t) * H + h) * (long long)D); };
    auto vrow = [&](int t) { return v + 2 * (((b * S + t0 + t) * H + h) * (long long)D); };
    stage_tile64(ks, krow, D, cnt);
    stage_tile64(vs, vrow, D, cnt);
    __syncthreads();
    uint16_t* kmx = kmax_part + (bh * tiles + z) * D;
    uint16_t* vmx = vmax_part + (bh * tiles + z) * D;
    if (cnt == PF_BLK) {
        k_emit_block64<true>(ks, k_first_8, k_mid_4, k_last_4, bh * nmb + z, D, kmx);
        // V rows: 64 tokens x D/32 pieces
        const int per_tok = D >> 5;
        for (int i = threadIdx.x; i < PF_BLK * per_tok; i += blockDim.x) {
            const int t = i / per_tok, c = i - t * per_tok;
            const size_t prow = (size_t)bh * max_seq_len + t0 + t;
            const uint4* src = reinterpret_cast<const uint4*>(vs + t * pitch + c * 64);      // shared memory
            v_write32(src[0], src[1], src[2], src[3], v_first_8 + prow * D + c * 32, v_mid_4 + prow * (D >> 1) + c * 16,
                      v_last_4 + prow * (D >> 1) + c * 16);
        }
    } else {
        // the prompt's last, partial tile stays in fp16 (residual buffers [B,64,H,D], rows 0..cnt-1)
        const int vec_per_row = pitch >> 4;
        for (int i = threadIdx.x; i < cnt * vec_per_row; i += blockDim.x) {
            const int t = i / vec_per_row, vv = i - t * vec_per_row;
            const size_t dst = 2 * ((((size_t)b * PF_BLK + t) * H + h) * (size_t)D) + vv * 16;
            *reinterpret_cast<uint4*>(restk + dst) = *reinterpret_cast<const uint4*>(ks + t * pitch + vv * 16);
            *reinterpret_cast<uint4*>(restv + dst) = *reinterpret_cast<const uint4*>(vs + t * pitch + vv * 16);
        }
    }
    // per-channel signed maxima of the tile (K's come out of the block writer when the tile is whole)
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float vm = -INFINITY, km = -INFINITY;
        for (int t = 0; t < cnt; ++t) {
            vm = fmaxf(vm, __half2float(*reinterpret_cast<const __half*>(vs + t * pitch + 2 * d)));
            if (cnt != PF_BLK) km = fmaxf(km, __half2float(*reinterpret_cast<const __half*>(ks + t * pitch + 2 * d)));
        }
        vmx[d] = __half_as_ushort(__float2half_rn(vm));
        if (cnt != PF_BLK) kmx[d] = __half_as_ushort(__float2half_rn(km));
    }
}

// exponent field of the signed maximum over the tiles -> [B,1,H,D] bytes
__global__ void __launch_bounds__(128)
exp_reduce_kernel(const uint16_t* __restrict__ kmax_part, const uint16_t* __restrict__ vmax_part,
                  uint8_t* __restrict__ k_exp, uint8_t* __restrict__ v_exp, int D, int tiles) {
    const long long bh = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float km = -INFINITY, vm = -INFINITY;
        for (int z = 0; z < tiles; ++z) {
            km = fmaxf(km, __half2float(__ushort_as_half(kmax_part[(bh * tiles + z) * D + d])));
            vm = fmaxf(vm, __half2float(__ushort_as_half(vmax_part[(bh * tiles + z) * D + d])));
        }
        k_exp[bh * D + d] = (uint8_t)((__half_as_ushort(__float2half_rn(km)) >> 10) & 0x1Fu);
        v_exp[bh * D + d] = (uint8_t)((__half_as_ushort(__float2half_rn(vm)) >> 10) & 0x1Fu);
    }
}

}  // namespace akv

using namespace akv;

extern "C" {

long long akv_prefill_scratch_bytes(int bsz, int n_kv_heads, int head_dim, int seqlen) {
    if (bsz <= 0 || n_kv_heads <= 0 || head_dim <= 0 || seqlen <= 0) return -1;
    const long long tiles = (seqlen + PF_BLK - 1) / PF_BLK;
    return 2ll * bsz * n_kv_heads * tiles * head_dim * 2;
}

int akv_prefill(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* k, const void* v,
                void* scratch, long long scratch_bytes, int bsz, int n_kv_heads, int head_dim, int max_seq_len,
                int seqlen, void* stream) {
    set_error("");
    const int B = bsz, H = n_kv_heads, D = head_dim, S = seqlen;
    AKV_REQUIRE(k_first_8 && k_mid_4 && k_last_4 && v_first_8 && v_mid_4 && v_last_4 && k_exp_max && v_exp_max &&
                restk && restv && k && v && scratch, AKV_ERR_NULL, "prefill: null pointer");
    AKV_REQUIRE(B > 0 && B <= 65535 && H > 0 && H <= 65535 && D > 0 && D % 32 == 0 && D <= 256 && S > 0 &&
                S <= max_seq_len, AKV_ERR_SHAPE, "prefill: unsupported extent (bsz %d, heads %d, head_dim %d [multiple "
                "of 32, at most 256], seqlen %d, max_seq_len %d)", B, H, D, S, max_seq_len);
    AKV_REQUIRE(scratch_bytes >= akv_prefill_scratch_bytes(B, H, D, S), AKV_ERR_SHAPE,
                "prefill: scratch of %lld bytes is too small", scratch_bytes);
    AKV_REQUIRE(aligned16(k_first_8) && aligned16(k_mid_4) && aligned16(k_last_4) && aligned16(v_first_8) &&
                aligned16(v_mid_4) && aligned16(v_last_4) && aligned16(restk) && aligned16(restv) && aligned16(k) &&
                aligned16(v) && aligned16(scratch), AKV_ERR_ALIGN, "prefill: pointers must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int tiles = (S + PF_BLK - 1) / PF_BLK;
    const int nmb = (max_seq_len + PF_BLK - 1) / PF_BLK;
    uint16_t* kmax_part = static_cast<uint16_t*>(scratch);
    uint16_t* vmax_part = kmax_part + (size_t)B * H * tiles * D;
    const size_t smem = (size_t)2 * PF_BLK * 2 * D;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_status(e, "prefill smem attribute");
    }
    dim3 grid(tiles, H, B);
    count_launch(2);
    prefill_kernel<<<grid, 128, smem, st>>>(
        static_cast<uint8_t*>(k_first_8), static_cast<uint8_t*>(k_mid_4), static_cast<uint8_t*>(k_last_4),
        static_cast<uint8_t*>(v_first_8), static_cast<uint8_t*>(v_mid_4), static_cast<uint8_t*>(v_last_4),
        static_cast<uint8_t*>(restk), static_cast<uint8_t*>(restv), static_cast<const uint8_t*>(k),
        static_cast<const uint8_t*>(v), kmax_part, vmax_part, H, D, S, nmb, max_seq_len, tiles);
    int rc = cuda_status(cudaGetLastError(), "prefill launch");
    if (rc != AKV_OK) return rc;
    exp_reduce_kernel<<<B * H, 128, 0, st>>>(kmax_part, vmax_part, static_cast<uint8_t*>(k_exp_max),
                                            static_cast<uint8_t*>(v_exp_max), D, tiles);
    return cuda_status(cudaGetLastError(), "prefill reduce launch");
}

}  // extern "C"
