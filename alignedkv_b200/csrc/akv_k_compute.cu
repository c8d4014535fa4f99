// Precision-aligned q.K^T over the quantized K blocks.
//
// Replaces the reference's k_cache_compute_kernel (extension/csrc/K_cache.cu:174-310).  Results are
// bit-identical: every token's score is the fp16 fused-multiply-add chain over channels 0..D-1 followed by one
// fp16 multiply with half(sqrt_dim), and a nibble plane that the alignment rule skips is replaced by the same
// constants (K_cache.cu:201-205,249-252).
//
// Design (B200): the kernel is a pure HBM stream, so it is organised around keeping ~100 KB of loads in flight
// per SM.  Each WARP owns a private ring of shared-memory stages that it fills with 16-byte asynchronous copies
// and drains itself - no block-level barrier exists.  A warp works on units of 4 consecutive 64-token blocks of
// one (batch, head); a stage holds 16 channels of those 4 blocks: 4 x 1 KB of the high-byte plane plus, only for
// the channels whose alignment code asks for them, the 32-byte rows of the mid / low nibble planes.  The plane
// bytes that are skipped are never requested from memory.  Lane (tile, i) owns tokens 8i..8i+7 of its tile and
// keeps four fp16x2 accumulators, so one 8-byte and two 4-byte shared loads feed four FMAs and no cross-lane
// reduction is needed (which is what keeps the channel-order fp16 sum exact).
#include "akv_common.cuh"

namespace akv {

namespace kc {
constexpr int KCH = 16;                          // channels per stage
constexpr int TILES = 4;                         // 64-token blocks per warp unit
constexpr int F_TILE = KCH * 64 + 64;            // 1088: +64 staggers tiles across shared-memory banks
constexpr int N_TILE = KCH * 32 + 32;            // 544
constexpr int F_BYTES = TILES * F_TILE;          // 4352
constexpr int N_BYTES = TILES * N_TILE;          // 2176
constexpr int STAGE = F_BYTES + 2 * N_BYTES;     // 8704
constexpr int MAX_D = 256;
constexpr int META = 2 * MAX_D + MAX_D + 64;     // q halves + kq bytes + masks (16 words)
constexpr int NMETA = 3;
}  // namespace kc

struct KParams {
    const uint8_t* first8;
    const uint8_t* mid4;
    const uint8_t* last4;
    const uint8_t* kq;
    const uint8_t* kqmax;
    const uint8_t* q;
    uint8_t* s;
    int BH, nb, nmb, D, ngroups;
    long long units;
    uint32_t scale2;  // half(sqrt_dim) in both halves
    int reference;
};

__device__ __forceinline__ void k_unit_coords(const KParams& p, long long u, int& bh, int& g) {
    bh = (int)(u / p.ngroups);
    g = (int)(u - (long long)bh * p.ngroups);
}

template <int STAGES>
__global__ void __launch_bounds__(256, 1) k_compute_kernel(const KParams p) {
    using namespace kc;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wpc = blockDim.x >> 5;
    const long long W = (long long)gridDim.x * wpc;
    const long long w = (long long)blockIdx.x * wpc + warp;
    if (w >= p.units) return;
    const long long my_units = (p.units - w + W - 1) / W;
    const int nch = p.D / KCH;
    const long long total = my_units * nch;

    uint8_t* ring = smem + (size_t)warp * (STAGES * STAGE + NMETA * META);
    uint8_t* meta0 = ring + STAGES * STAGE;
    const uint32_t ring_a = smem_u32(ring);
    const uint32_t meta_a = smem_u32(meta0);

    // ---- metadata of a unit: q row, kq row (async) and the kqmax byte (register)
    auto prefetch_meta = [&](long long k) -> uint32_t {
        int bh, g;
        k_unit_coords(p, w + k * W, bh, g);
        const uint32_t m = meta_a + (uint32_t)(k % NMETA) * META;
        const int qv = p.D >> 3;   // 16-byte pieces of the q row (2*D bytes)
        const int kv = p.D >> 4;   // 16-byte pieces of the kq row
        if (lane < qv) cp_async16(m + lane * 16, p.q + (size_t)bh * 2 * p.D + lane * 16);
        if (lane < kv) cp_async16(m + 2 * MAX_D + lane * 16, p.kq + (size_t)bh * p.D + lane * 16);
        return (uint32_t)__ldg(p.kqmax + bh);
    };
    // ---- alignment masks of unit k from its staged kq row: bit d of mid/last mask = plane row d is read
    auto build_masks = [&](long long k, uint32_t top) {
        uint8_t* m = meta0 + (size_t)(k % NMETA) * META;
        uint32_t* masks = reinterpret_cast<uint32_t*>(m + 3 * MAX_D);
        for (int r = 0; r < (p.D + 31) / 32; ++r) {
            int d = r * 32 + lane;
            uint32_t diff = 0;
            if (d < p.D) diff = (top - (uint32_t)m[2 * MAX_D + d]) & 0xFFu;
            uint32_t mm = __ballot_sync(0xFFFFFFFFu, p.reference || diff < 8);
            uint32_t lm = __ballot_sync(0xFFFFFFFFu, p.reference || diff < 4);
            if (lane == 0) {
                masks[r] = mm;
                masks[8 + r] = lm;
            }
        }
        __syncwarp();
    };

    uint32_t top_next = 0;
    // ---- producer: stage item j = (unit k, channel chunk c)
    auto issue = [&](long long j) {
        const long long k = j / nch;
        const int c = (int)(j - k * nch);
        if (c == 0) {
            const uint32_t top = top_next;
            build_masks(k, top);
            if (k + 1 < my_units) top_next = prefetch_meta(k + 1);
        }
        int bh, g;
        k_unit_coords(p, w + k * W, bh, g);
        const uint32_t* masks = reinterpret_cast<const uint32_t*>(meta0 + (size_t)(k % NMETA) * META + 3 * MAX_D);
        const uint32_t mm = (masks[c >> 1] >> ((c & 1) * 16)) & 0xFFFFu;
        const uint32_t lm = (masks[8 + (c >> 1)] >> ((c & 1) * 16)) & 0xFFFFu;
        const uint32_t st = ring_a + (uint32_t)(j % STAGES) * STAGE;
        const int blk0 = g * TILES;
        const size_t tile0 = ((size_t)bh * p.nmb + blk0) * p.D + (size_t)c * KCH;  // row index of (blk0, c*16)
#pragma unroll
        for (int it = 0; it < 8; ++it) {  // high-byte plane: 4 tiles x 1 KB
            const int t = it >> 1;
            const int off = (((it & 1) << 5) + lane) << 4;
            if (blk0 + t < p.nb)
                cp_async16(st + t * F_TILE + off, p.first8 + (tile0 + (size_t)t * p.D) * 64 + off);
        }
        const int row = lane >> 1, half = (lane & 1) << 4;
        const bool need_m = (mm >> row) & 1u, need_l = (lm >> row) & 1u;
#pragma unroll
        for (int t = 0; t < TILES; ++t) {  // nibble planes: only the rows the alignment rule reads
            if (blk0 + t < p.nb) {
                const size_t src = (tile0 + (size_t)t * p.D + row) * 32 + half;
                if (need_m) cp_async16(st + F_BYTES + t * N_TILE + row * 32 + half, p.mid4 + src);
                if (need_l) cp_async16(st + F_BYTES + N_BYTES + t * N_TILE + row * 32 + half, p.last4 + src);
            }
        }
    };

    // ---- prologue
    top_next = prefetch_meta(0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
    for (int j = 0; j < STAGES - 1; ++j) {
        if (j < total) issue(j);
        cp_async_commit();
    }

    const int tile = lane >> 3, li = lane & 7;
    uint32_t acc02 = 0, acc13 = 0, acc46 = 0, acc57 = 0;
    for (long long i = 0; i < total; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        if (i + STAGES - 1 < total) issue(i + STAGES - 1);
        cp_async_commit();

        const long long k = i / nch;
        const int c = (int)(i - k * nch);
        const uint32_t m = meta_a + (uint32_t)(k % NMETA) * META;
        const uint32_t mm = (lds32(m + 3 * MAX_D + (c >> 1) * 4) >> ((c & 1) * 16)) & 0xFFFFu;
        const uint32_t lm = (lds32(m + 3 * MAX_D + 32 + (c >> 1) * 4) >> ((c & 1) * 16)) & 0xFFFFu;
        const uint32_t st = ring_a + (uint32_t)(i % STAGES) * STAGE;
        const uint32_t fa = st + tile * F_TILE + li * 8;
        const uint32_t ma = st + F_BYTES + tile * N_TILE + li * 4;
        const uint32_t la = ma + N_BYTES;
        const uint32_t qa = m + c * (KCH * 2);
#pragma unroll
        for (int r = 0; r < KCH; ++r) {
            const uint2 f = lds64(fa + r * 64);
            uint32_t M = 0x88888888u, L = 0u;        // neither nibble plane read: low byte becomes 0x80
            if ((mm >> r) & 1u) {                    // warp-uniform
                M = lds32(ma + r * 32);
                L = 0x88888888u;                     // low plane skipped: low nibble becomes 8
                if ((lm >> r) & 1u) L = lds32(la + r * 32);
            }
            const uint32_t lbe = (M & 0xF0F0F0F0u) | ((L >> 4) & 0x0F0F0F0Fu);   // low bytes of tokens 0,2,4,6
            const uint32_t lbo = ((M << 4) & 0xF0F0F0F0u) | (L & 0x0F0F0F0Fu);   // low bytes of tokens 1,3,5,7
            const uint32_t qh = lds16(qa + r * 2);
            const uint32_t q2 = qh | (qh << 16);
            acc02 = hfma2_bits(__byte_perm(lbe, f.x, 0x6140), q2, acc02);
            acc13 = hfma2_bits(__byte_perm(lbo, f.x, 0x7150), q2, acc13);
            acc46 = hfma2_bits(__byte_perm(lbe, f.y, 0x6342), q2, acc46);
            acc57 = hfma2_bits(__byte_perm(lbo, f.y, 0x7352), q2, acc57);
        }
        if (c == nch - 1) {  // unit finished: scale, reorder to token order, one 16-byte store per lane
            int bh, g;
            k_unit_coords(p, w + k * W, bh, g);
            const int blk = g * TILES + tile;
            if (blk < p.nb) {
                acc02 = hmul2_bits(acc02, p.scale2);
                acc13 = hmul2_bits(acc13, p.scale2);
                acc46 = hmul2_bits(acc46, p.scale2);
                acc57 = hmul2_bits(acc57, p.scale2);
                uint4 o;
                o.x = __byte_perm(acc02, acc13, 0x5410);
                o.y = __byte_perm(acc02, acc13, 0x7632);
                o.z = __byte_perm(acc46, acc57, 0x5410);
                o.w = __byte_perm(acc46, acc57, 0x7632);
                const size_t row = (size_t)bh * (size_t)(p.nb + 1) * 64 + (size_t)blk * 64 + li * 8;
                *reinterpret_cast<uint4*>(p.s + row * 2) = o;
            }
            acc02 = acc13 = acc46 = acc57 = 0;
        }
    }
    cp_async_wait<0>();
}

// Any block length / head size: one thread per token, planes read straight from global memory.
__global__ void __launch_bounds__(128)
k_compute_generic_kernel(const uint8_t* __restrict__ first8, const uint8_t* __restrict__ mid4,
                         const uint8_t* __restrict__ last4, const uint8_t* __restrict__ kq,
                         const uint8_t* __restrict__ kqmax, const __half* __restrict__ q, __half* __restrict__ s,
                         int nb, int nmb, int D, int d_block, __half scale, int reference, long long total) {
    const int hb = d_block >> 1;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int t = (int)(i % d_block);
        long long r = i / d_block;
        int z = (int)(r % nb);
        long long bh = r / nb;
        const uint32_t top = kqmax[bh];
        __half acc = __ushort_as_half(0);
        for (int d = 0; d < D; ++d) {
            uint32_t diff = (top - (uint32_t)kq[bh * D + d]) & 0xFFu;
            long long row = ((bh * nmb + z) * D + d) * hb;
            uint32_t f = first8[2 * row + t];
            uint32_t mb = 0x88u, lb = 0x00u;
            if (reference || diff < 8) {
                mb = mid4[row + (t >> 1)];
                lb = (reference || diff < 4) ? (uint32_t)last4[row + (t >> 1)] : 0x88u;
            }
            uint32_t bits = (t & 1) ? ((f << 8) + ((mb & 0x0Fu) << 4) + (lb & 0x0Fu))
                                    : ((f << 8) + (mb & 0xF0u) + ((lb & 0xF0u) >> 4));
            acc = __hfma(__ushort_as_half((unsigned short)bits), q[bh * D + d], acc);
        }
        s[bh * (long long)(nb + 1) * d_block + (long long)z * d_block + t] = __hmul(acc, scale);
    }
}

int launch_k_compute(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* kq,
                     const uint8_t* kqmax, const uint8_t* q, uint8_t* s, int bsz, int H, int nb, int nmb, int D,
                     int d_block, float sqrt_dim, int reference, cudaStream_t st) {
    using namespace kc;
    const __half scale = __float2half_rn(sqrt_dim);
    const bool fast = d_block == 64 && D % 16 == 0 && D >= 64 && D <= MAX_D && aligned16(first8) &&
                      aligned16(mid4) && aligned16(last4) && aligned16(kq) && aligned16(q) && aligned16(s);
    if (!fast) {
        long long total = (long long)bsz * H * nb * d_block;
        long long want = (total + 127) / 128;
        int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
        k_compute_generic_kernel<<<grid, 128, 0, st>>>(first8, mid4, last4, kq, kqmax,
                                                       reinterpret_cast<const __half*>(q),
                                                       reinterpret_cast<__half*>(s), nb, nmb, D, d_block, scale,
                                                       reference, total);
        return cuda_status(cudaGetLastError(), "k_cache_compute launch");
    }
    KParams p;
    p.first8 = first8; p.mid4 = mid4; p.last4 = last4; p.kq = kq; p.kqmax = kqmax; p.q = q; p.s = s;
    p.BH = bsz * H; p.nb = nb; p.nmb = nmb; p.D = D;
    p.ngroups = (nb + TILES - 1) / TILES;
    p.units = (long long)p.BH * p.ngroups;
    const unsigned short sb = __half_as_ushort(scale);
    p.scale2 = (uint32_t)sb | ((uint32_t)sb << 16);
    p.reference = reference;

    // Pick warps per CTA (one CTA per SM) so that the last wave of units is as full as possible, then give
    // each warp as many ring stages as the shared memory allows.
    const int sms = sm_count();
    const int budget = max_dyn_smem();
    int best_wpc = 8;
    double best_eff = -1.0;
    for (int wpc = 8; wpc >= 5; --wpc) {
        long long Wt = (long long)sms * wpc;
        long long waves = (p.units + Wt - 1) / Wt;
        double eff = (double)p.units / (double)(waves * Wt);
        if (eff > best_eff + 0.02) { best_eff = eff; best_wpc = wpc; }
    }
    int wpc = best_wpc;
    long long ctas = (p.units + wpc - 1) / wpc;
    int grid = (int)(ctas < sms ? ctas : sms);
    int per_warp = budget / wpc;
    int stages = (per_warp - NMETA * META) / STAGE;
    if (stages > 4) stages = 4;
    AKV_REQUIRE(stages >= 3, AKV_ERR_CUDA, "k_cache_compute: %d bytes of shared memory are too few", budget);
    size_t smem = (size_t)wpc * (stages * STAGE + NMETA * META);
    cudaError_t e;
    if (stages == 4) {
        e = cudaFuncSetAttribute(k_compute_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_status(e, "k_cache_compute smem attribute");
        k_compute_kernel<4><<<grid, wpc * 32, smem, st>>>(p);
    } else {
        e = cudaFuncSetAttribute(k_compute_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_status(e, "k_cache_compute smem attribute");
        k_compute_kernel<3><<<grid, wpc * 32, smem, st>>>(p);
    }
    return cuda_status(cudaGetLastError(), "k_cache_compute launch");
}

}  // namespace akv
