// Precision-aligned q.K^T over the quantized K blocks.
//
// Replaces the reference's k_cache_compute_kernel (extension/csrc/K_cache.cu:174-310).  Results are
// bit-identical: every token's score is the fp16 fused-multiply-add chain over channels 0..D-1 followed by one
// fp16 multiply with half(sqrt_dim), and a nibble plane that the alignment rule skips is replaced by the same
// constants (K_cache.cu:201-205,249-252).
//
// Design (B200): the kernel is a pure HBM stream.  Each WARP owns a private ring of shared-memory stages that
// it fills with 16-byte asynchronous copies and drains itself - no block-level barrier exists.  A warp works
// through a contiguous run of units; a unit is 4 consecutive 64-token blocks of one (batch, head), and a stage
// holds KCH channels of those 4 blocks: the high-byte rows plus, only for the channels whose alignment code
// asks for them, the 32-byte rows of the mid / low nibble planes (rows that are skipped are never requested
// from memory; the producer writes the substitute constants into their slots so that the consumer is
// branch-free).  Lane (tile, i) owns tokens 8i..8i+7 of its tile and keeps four fp16x2 accumulators: one 8-byte
// and two 4-byte shared loads feed four FMAs, and no cross-lane reduction exists, which is what keeps the
// channel-order fp16 sum exact.  Grouped-query attention (G query heads per KV head) runs the G passes over a
// unit's tiles back to back on the same warp, so that only the first pass reads HBM.
#include "akv_common.cuh"

namespace akv {

namespace kc {
constexpr int TILES = 4;                         // 64-token blocks per warp unit
constexpr int MAX_D = 256;
constexpr int META = 64 + 4 * MAX_D;             // plane-read masks (16 words) + q as duplicated fp16x2 words
constexpr int NMETA = 3;
__host__ __device__ constexpr int f_tile(int kch) { return kch * 64 + 64; }   // +64: tiles land on distinct banks
__host__ __device__ constexpr int n_tile(int kch) { return kch * 32 + 32; }
__host__ __device__ constexpr int stage_bytes(int kch) { return TILES * f_tile(kch) + 2 * TILES * n_tile(kch); }
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
    int G;                // query heads per KV head; kq, kqmax, q and s are per (batch, query head)
    int units, upw;       // total units, units per warp (contiguous run)
    uint32_t scale2;      // half(sqrt_dim) in both halves
    int reference;
};

__device__ __forceinline__ void st_shared_v4(uint32_t a, uint32_t v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(a), "r"(v) : "memory");
}

// Position of a stream of stages (unit, channel chunk) inside one warp's run of units.  Units are ordered
// (batch, KV head) -> group of 4 blocks -> query head of the group, so the G passes over the same tiles (one per
// query head) run back to back on the same warp and all but the first are served by L2.
struct KCursor {
    int u, g, bh, gq, c;      // absolute unit, block group inside (batch, KV head), (batch, KV head), query head, chunk
    int slot;                 // metadata slot of the current (batch, query head)
    size_t row;               // plane row index of (tile 0 of the unit, first channel of the chunk)
};

template <int KCH, int STAGES>
__global__ void __launch_bounds__(512, 1) k_compute_kernel(const KParams p) {
    using namespace kc;
    constexpr int F_TILE = f_tile(KCH), N_TILE = n_tile(KCH);
    constexpr int F_BYTES = TILES * F_TILE, N_BYTES = TILES * N_TILE, STAGE = F_BYTES + 2 * N_BYTES;
    constexpr int F_IT = KCH / 8;                 // 16-byte copies per lane and tile for the high-byte plane
    constexpr int ROW_LANES = 2 * KCH;            // lanes that cover the nibble rows of one tile
    constexpr int TILES_PER_IT = 32 / ROW_LANES;  // 1 (KCH 16) or 2 (KCH 8)
    static_assert(KCH == 8 || KCH == 16, "channels per stage");
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_enter();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wpc = blockDim.x >> 5;
    const int w = blockIdx.x * wpc + warp;
    const int u_begin = w * p.upw;
    if (u_begin >= p.units) return;
    const int u_end = (u_begin + p.upw < p.units) ? u_begin + p.upw : p.units;
    const int nch = p.D / KCH;
    const int total = (u_end - u_begin) * nch;
    const size_t tile_f = (size_t)p.D * 64, tile_n = (size_t)p.D * 32;
    const int G = p.G;

    uint8_t* ring = smem + (size_t)warp * (STAGES * STAGE + NMETA * META);
    uint8_t* meta0 = ring + STAGES * STAGE;
    const uint32_t ring_a = smem_u32(ring);

    auto cursor_at = [&](int u) {
        KCursor k;
        k.u = u;
        k.gq = u % G;
        const int ug = u / G;
        k.bh = ug / p.ngroups;
        k.g = ug - k.bh * p.ngroups;
        k.c = 0;
        k.slot = 0;
        k.row = ((size_t)k.bh * p.nmb + (size_t)k.g * TILES) * p.D;
        return k;
    };
    auto advance = [&](KCursor& k) {   // next stage; returns true when a new (batch, query head) starts
        k.row += KCH;
        if (++k.c < nch) return false;
        k.c = 0;
        ++k.u;
        if (++k.gq < G) {                                 // same tiles again for the next query head of the group
            k.row -= (size_t)p.D;
            k.slot = (k.slot + 1 == NMETA) ? 0 : k.slot + 1;
            return true;
        }
        k.gq = 0;
        if (++k.g < p.ngroups) {
            k.row += (size_t)(TILES - 1) * p.D;          // next 4 tiles of the same (batch, KV head)
            if (G == 1) return false;
            k.slot = (k.slot + 1 == NMETA) ? 0 : k.slot + 1;
            return true;
        }
        k.g = 0;
        ++k.bh;
        k.slot = (k.slot + 1 == NMETA) ? 0 : k.slot + 1;
        k.row = (size_t)k.bh * p.nmb * p.D;
        return true;
    };
    // Per (batch, query head): plane-read masks (bit d set = row d of that plane is read: mid iff
    // (u8)(kqmax - kq[d]) < 8, low iff < 4; K_cache.cu:211,249-250) and q as fp16x2 words with both halves equal.
    auto load_meta = [&](long long bhq, int slot) {
        uint32_t* masks = reinterpret_cast<uint32_t*>(meta0 + (size_t)slot * META);
        uint32_t* q2 = masks + 16;
        const uint32_t top = __ldg(p.kqmax + bhq);
        for (int r = 0; r < (p.D + 31) / 32; ++r) {
            const int d = r * 32 + lane;
            uint32_t diff = 0, qh = 0;
            if (d < p.D) {
                diff = (top - (uint32_t)__ldg(p.kq + (size_t)bhq * p.D + d)) & 0xFFu;
                qh = __ldg(reinterpret_cast<const uint16_t*>(p.q) + (size_t)bhq * p.D + d);
                q2[d] = qh | (qh << 16);
            }
            const uint32_t mm = __ballot_sync(0xFFFFFFFFu, p.reference || diff < 8);
            const uint32_t lm = __ballot_sync(0xFFFFFFFFu, p.reference || diff < 4);
            if (lane == 0) {
                masks[r] = mm;
                masks[8 + r] = lm;
            }
        }
        __syncwarp();
    };

    const int nrow = (lane % ROW_LANES) >> 1, nhalf = (lane & 1) << 4, ntsub = lane / ROW_LANES;

    // ---- producer: async copies of one stage
    KCursor pk = cursor_at(u_begin);
    int pstage = 0;
    auto issue = [&]() {
        const uint32_t* masks = reinterpret_cast<const uint32_t*>(meta0 + (size_t)pk.slot * META);
        const int sh = ((pk.c * KCH) & 31) + nrow, wi = (pk.c * KCH) >> 5;
        const bool need_m = (masks[wi] >> sh) & 1u;
        const bool need_l = (masks[8 + wi] >> sh) & 1u;
        const uint32_t st = ring_a + (uint32_t)pstage * STAGE;
        const int ptiles = p.nb - pk.g * TILES;
        const uint8_t* pf = p.first8 + pk.row * 64 + lane * 16;
#pragma unroll
        for (int it = 0; it < TILES * F_IT; ++it) {      // high-byte plane: KCH*64 contiguous bytes per tile
            const int t = it / F_IT, v = it % F_IT;
            if (t < ptiles) cp_async16(st + t * F_TILE + v * 512 + lane * 16, pf + t * tile_f + v * 512);
        }
        const size_t pn = (pk.row + nrow) * 32 + nhalf;
        const uint32_t nd = st + F_BYTES + nrow * 32 + nhalf;
#pragma unroll
        for (int it = 0; it < TILES / TILES_PER_IT; ++it) {   // nibble planes: rows the rule reads, else constants
            const int t = it * TILES_PER_IT + ntsub;
            if (t < ptiles) {
                const uint32_t dm = nd + t * N_TILE, dl = dm + N_BYTES;
                if (need_m) cp_async16(dm, p.mid4 + pn + t * tile_n);
                else st_shared_v4(dm, 0x88888888u);              // plane not read: low byte becomes 0x80
                if (need_l) cp_async16(dl, p.last4 + pn + t * tile_n);
                else st_shared_v4(dl, need_m ? 0x88888888u : 0u);  // low plane not read: low nibble becomes 8
            }
        }
        pstage = (pstage + 1 == STAGES) ? 0 : pstage + 1;
        if (advance(pk) && pk.u < u_end) load_meta((long long)pk.bh * G + pk.gq, pk.slot);
    };

    // ---- prologue
    load_meta((long long)pk.bh * G + pk.gq, 0);
    for (int j = 0; j < STAGES - 1; ++j) {
        if (j < total) issue();
        cp_async_commit();
    }

    const int tile = lane >> 3, li = lane & 7;
    uint32_t acc02 = 0, acc13 = 0, acc46 = 0, acc57 = 0;
    KCursor ck = cursor_at(u_begin);
    int cstage = 0;
    for (int i = 0; i < total; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        if (i + STAGES - 1 < total) issue();
        cp_async_commit();

        const uint8_t* stp = ring + (size_t)cstage * STAGE;
        cstage = (cstage + 1 == STAGES) ? 0 : cstage + 1;
        const uint2* fp = reinterpret_cast<const uint2*>(stp + tile * F_TILE + li * 8);
        const uint32_t* mp = reinterpret_cast<const uint32_t*>(stp + F_BYTES + tile * N_TILE + li * 4);
        const uint32_t* lp = reinterpret_cast<const uint32_t*>(stp + F_BYTES + N_BYTES + tile * N_TILE + li * 4);
        const uint4* qp = reinterpret_cast<const uint4*>(meta0 + (size_t)ck.slot * META + 64 + ck.c * (KCH * 4));
#pragma unroll
        for (int r4 = 0; r4 < KCH / 4; ++r4) {
            const uint4 qv = qp[r4];
            const uint32_t q2s[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) {
                const int r = r4 * 4 + rr;
                const uint2 f = fp[r * 8];
                const uint32_t M = mp[r * 8], L = lp[r * 8];
                const uint32_t lbe = (M & 0xF0F0F0F0u) | ((L >> 4) & 0x0F0F0F0Fu);   // low bytes, tokens 0,2,4,6
                const uint32_t lbo = ((M << 4) & 0xF0F0F0F0u) | (L & 0x0F0F0F0Fu);   // low bytes, tokens 1,3,5,7
                acc02 = hfma2_bits(__byte_perm(lbe, f.x, 0x6140), q2s[rr], acc02);
                acc13 = hfma2_bits(__byte_perm(lbo, f.x, 0x7150), q2s[rr], acc13);
                acc46 = hfma2_bits(__byte_perm(lbe, f.y, 0x6342), q2s[rr], acc46);
                acc57 = hfma2_bits(__byte_perm(lbo, f.y, 0x7352), q2s[rr], acc57);
            }
        }
        const long long cbhq = (long long)ck.bh * G + ck.gq;
        const int cg = ck.g;
        const bool last_chunk = (ck.c == nch - 1);
        advance(ck);
        if (last_chunk) {  // unit finished: scale, reorder to token order, one 16-byte store per lane
            const int blk = cg * TILES + tile;
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
                const size_t row = (size_t)cbhq * (size_t)(p.nb + 1) * 64 + (size_t)blk * 64 + li * 8;
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
                         int nb, int nmb, int D, int d_block, int G, __half scale, int reference, long long total) {
    const int hb = d_block >> 1;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int t = (int)(i % d_block);
        long long r = i / d_block;
        int z = (int)(r % nb);
        long long bh = r / nb;            // (batch, query head)
        const long long bkv = bh / G;     // (batch, KV head)
        const uint32_t top = kqmax[bh];
        __half acc = __ushort_as_half(0);
        for (int d = 0; d < D; ++d) {
            uint32_t diff = (top - (uint32_t)kq[bh * D + d]) & 0xFFu;
            long long row = ((bkv * nmb + z) * D + d) * hb;
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

// q.K^T over nb quantized blocks.  H = KV heads, group = query heads per KV head; kq, kqmax, q and the score rows are
// per (batch, query head) with query head = KV head * group + g.
int launch_k_compute(const uint8_t* first8, const uint8_t* mid4, const uint8_t* last4, const uint8_t* kq,
                     const uint8_t* kqmax, const uint8_t* q, uint8_t* s, int bsz, int H, int group, int nb, int nmb,
                     int D, int d_block, float sqrt_dim, int reference, cudaStream_t st) {
    using namespace kc;
    const __half scale = __float2half_rn(sqrt_dim);
    const bool fast = d_block == 64 && D % 16 == 0 && D >= 64 && D <= MAX_D && aligned16(first8) &&
                      aligned16(mid4) && aligned16(last4) && aligned16(kq) && aligned16(q) && aligned16(s);
    if (!fast) {
        long long total = (long long)bsz * H * group * nb * d_block;
        long long want = (total + 127) / 128;
        int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
        k_compute_generic_kernel<<<grid, 128, 0, st>>>(first8, mid4, last4, kq, kqmax,
                                                       reinterpret_cast<const __half*>(q),
                                                       reinterpret_cast<__half*>(s), nb, nmb, D, d_block, group,
                                                       scale, reference, total);
        return cuda_status(cudaGetLastError(), "k_cache_compute launch");
    }
    KParams p;
    p.first8 = first8; p.mid4 = mid4; p.last4 = last4; p.kq = kq; p.kqmax = kqmax; p.q = q; p.s = s;
    p.BH = bsz * H; p.nb = nb; p.nmb = nmb; p.D = D;
    p.ngroups = (nb + TILES - 1) / TILES;
    p.G = group;
    const long long units = (long long)p.BH * p.ngroups * group;
    AKV_REQUIRE(units < (1ll << 30), AKV_ERR_OVERFLOW, "k_cache_compute: too many blocks");
    p.units = (int)units;
    const unsigned short sb = __half_as_ushort(scale);
    p.scale2 = (uint32_t)sb | ((uint32_t)sb << 16);
    p.reference = reference;

    // One CTA per SM.  Pick the channel-chunk size, ring depth and warps per CTA (tunable), trimming the warp
    // count so that every warp gets (nearly) the same whole number of units.
    const int sms = sm_count();
    const int budget = max_dyn_smem();
    const int kch = tuning().k_kch, stages = tuning().k_stages;
    const int per_warp = stages * stage_bytes(kch) + NMETA * META;
    int wmax = budget / per_warp;
    if (wmax > 16) wmax = 16;
    if (tuning().k_wpc > 0 && tuning().k_wpc < wmax) wmax = tuning().k_wpc;
    AKV_REQUIRE(wmax >= 1, AKV_ERR_CUDA, "k_cache_compute: %d bytes of shared memory are too few", budget);
    int wpc = wmax;
    double best_eff = -1.0;
    for (int c = wmax; c >= (wmax * 3 + 3) / 4; --c) {
        long long Wt = (long long)sms * c;
        long long upw = (units + Wt - 1) / Wt;
        double eff = (double)units / (double)(upw * Wt);
        if (eff > best_eff + 0.02) { best_eff = eff; wpc = c; }
    }
    {
        long long Wt = (long long)sms * wpc;
        p.upw = (int)((units + Wt - 1) / Wt);
    }
    const long long warps_needed = (units + p.upw - 1) / p.upw;
    int grid = (int)((warps_needed + wpc - 1) / wpc);
    size_t smem = (size_t)wpc * per_warp;
    auto go = [&](auto kern) -> int {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_status(e, "k_cache_compute smem attribute");
        launch_chained(kern, dim3(grid), dim3(wpc * 32), smem, st, p);
        return AKV_OK;
    };
    int rc;
    switch (kch * 10 + stages) {
        case 83: rc = go(k_compute_kernel<8, 3>); break;
        case 84: rc = go(k_compute_kernel<8, 4>); break;
        case 86: rc = go(k_compute_kernel<8, 6>); break;
        case 164: rc = go(k_compute_kernel<16, 4>); break;
        case 165: rc = go(k_compute_kernel<16, 5>); break;
        default: rc = go(k_compute_kernel<16, 3>); break;
    }
    if (rc != AKV_OK) return rc;
    return cuda_status(cudaGetLastError(), "k_cache_compute launch");
}

}  // namespace akv
