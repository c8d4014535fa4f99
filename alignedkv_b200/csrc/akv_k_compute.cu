// Precision-aligned q.K^T over the quantized K blocks.
//
// Replaces the reference's k_cache_compute_kernel (extension/csrc/K_cache.cu:174-310).  Results are
// bit-identical: every token's score is the fp16 fused-multiply-add chain over channels 0..D-1 followed by one
// fp16 multiply with half(sqrt_dim), and a nibble plane that the alignment rule skips is replaced by the same
// constants (K_cache.cu:201-205,249-252).
//
// Design (B200): the kernel is a pure HBM stream.  Each WARP owns a private ring of shared-memory stages that
// it fills with 16-byte asynchronous copies and drains itself - no block-level barrier exists.  A warp works
// through a contiguous run of units; a unit is 4 consecutive 64-token blocks of one (batch, KV head), and a stage
// holds KCH channels of those 4 blocks: the high-byte rows plus, only for the channels whose alignment code
// asks for them, the 32-byte rows of the mid / low nibble planes (rows that are skipped are never requested
// from memory).  Lane (tile, i) owns tokens 8i..8i+7 of its tile and keeps four fp16x2 accumulators per query head:
// one 8-byte and two 4-byte shared loads feed four FMAs, and no cross-lane reduction exists, which is what keeps the
// channel-order fp16 sum exact.
// Grouped-query attention (G query heads per KV head): a row is fetched when ANY head of the group needs it, every
// staged row is read from shared memory once and applied to the G heads in turn, each head substituting the
// reference's constants where its own code skips the plane - so plane bytes cross HBM once per group and the
// results equal G independent multi-head passes.  The byte shuffles that assemble a token's low byte from the
// nibble planes run on the half-rate integer pipe, and with them done per head the kernel was bound by that pipe
// (2.1 TB/s at G = 4).  So per row each lane assembles the low bytes once per alignment code (mid only / both planes;
// "neither" is a constant) and parks them in a private 8-byte slot per code of a small per-warp scratch; a head then
// fetches the pair of its own code with one 8-byte load whose offset (code x 256) was tabulated per (head, channel)
// when the (batch, KV head) started: one add and one load per head and row instead of selects and shuffles.  The
// rows are software-pipelined by one (two scratch buffers), so the store -> load round trip of a row overlaps the
// arithmetic of the previous one.  With G == 1 the producer writes the constants into the skipped rows' slots
// instead, and the consumer has neither selects nor scratch.
#include "akv_common.cuh"

namespace akv {

namespace kc {
constexpr int TILES = 4;                         // 64-token blocks per warp unit
constexpr int MAX_D = 256;
// Metadata slots per warp: the producer runs at most STAGES - 1 stages ahead of the consumer, which is less than one
// unit's stages, so it is at most one (batch, KV head) ahead: two slots.  (A third is kept for multi-head attention,
// whose slots are small and whose 16-channel stages make a unit only D/16 stages long.)
__host__ __device__ constexpr int nmeta(int G) { return G > 1 ? 2 : 3; }
__host__ __device__ constexpr int f_tile(int kch) { return kch * 64 + 64; }   // +64: tiles land on distinct banks
__host__ __device__ constexpr int n_tile(int kch) { return kch * 32 + 32; }
__host__ __device__ constexpr int stage_bytes(int kch) { return TILES * f_tile(kch) + 2 * TILES * n_tile(kch); }
}  // namespace kc

namespace kc {
// per (batch, KV head) metadata slot: union masks (16 words), then per query head D offset words (code x 256: which
// scratch slot holds the low bytes of the head's alignment code on that channel; used when G > 1) + D q words
__host__ __device__ constexpr int head_meta(int D) { return 8 * D; }
__host__ __device__ constexpr int meta_bytes(int D, int G) { return 64 + G * head_meta(D); }
// per-warp scratch of the grouped-query consumer: 2 row buffers x 3 codes x 32 lanes x 8 bytes
constexpr int SCR_CODE = 256, SCR_ROW = 3 * SCR_CODE, SCR_BYTES = 2 * SCR_ROW;
__host__ __device__ constexpr int scratch_bytes(int G) { return G > 1 ? SCR_BYTES : 0; }
}  // namespace kc

struct KParams {
    const uint8_t* first8;
    const uint8_t* mid4;
    const uint8_t* last4;
    const uint8_t* kq;
    const uint8_t* kqmax;
    const uint8_t* q;
    uint8_t* s;
    int BH, nb, nmb, D, ngroups;   // BH = batch x KV heads
    int units, upw;       // total units, units per warp (contiguous run)
    uint32_t scale2;      // half(sqrt_dim) in both halves
    int reference;
};

__device__ __forceinline__ void st_shared_v4(uint32_t a, uint32_t v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(a), "r"(v) : "memory");
}

// Position of a stream of stages (unit, channel chunk) inside one warp's run of units.
struct KCursor {
    int u, g, bh, c;          // absolute unit, block group inside (batch, KV head), (batch, KV head), channel chunk
    int slot;                 // metadata slot of the current (batch, KV head)
    size_t row;               // plane row index of (tile 0 of the unit, first channel of the chunk)
};

template <int KCH, int STAGES, int G>
__global__ void __launch_bounds__(G > 1 ? 256 : 512, 1) k_compute_kernel(const KParams p) {
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
    const int META = meta_bytes(p.D, G), HMETA = head_meta(p.D);

    constexpr int NMETA = nmeta(G);
    uint8_t* ring = smem + (size_t)warp * (STAGES * STAGE + NMETA * META + scratch_bytes(G));
    uint8_t* meta0 = ring + STAGES * STAGE;
    const uint32_t ring_a = smem_u32(ring);

    auto cursor_at = [&](int u) {
        KCursor k;
        k.u = u;
        k.bh = u / p.ngroups;
        k.g = u - k.bh * p.ngroups;
        k.c = 0;
        k.slot = 0;
        k.row = ((size_t)k.bh * p.nmb + (size_t)k.g * TILES) * p.D;
        return k;
    };
    auto advance = [&](KCursor& k) {   // next stage; returns true when a new (batch, KV head) starts
        k.row += KCH;
        if (++k.c < nch) return false;
        k.c = 0;
        ++k.u;
        if (++k.g < p.ngroups) {
            k.row += (size_t)(TILES - 1) * p.D;          // next 4 tiles of the same (batch, KV head)
            return false;
        }
        k.g = 0;
        ++k.bh;
        k.slot = (k.slot + 1 == NMETA) ? 0 : k.slot + 1;
        k.row = (size_t)k.bh * p.nmb * p.D;
        return true;
    };
    // Per (batch, KV head): for every query head of the group the plane-read masks (bit d set = row d of that plane
    // is read: mid iff (u8)(kqmax - kq[d]) < 8, low iff < 4; K_cache.cu:211,249-250) and q as fp16x2 words with
    // both halves equal; and the union of the masks, which is what the producer fetches.
    auto load_meta = [&](long long bh, int slot) {
        uint32_t* um = reinterpret_cast<uint32_t*>(meta0 + (size_t)slot * META);
        uint32_t u_mm[8], u_lm[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) u_mm[r] = u_lm[r] = 0;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const long long bhq = bh * G + g;
            uint32_t* offw = reinterpret_cast<uint32_t*>(meta0 + (size_t)slot * META + 64 + (size_t)g * HMETA);
            uint32_t* q2 = offw + p.D;
            const uint32_t top = __ldg(p.kqmax + bhq);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r * 32 >= p.D) break;
                const int d = r * 32 + lane;
                uint32_t diff = 0, qh = 0;
                if (d < p.D) {
                    diff = (top - (uint32_t)__ldg(p.kq + (size_t)bhq * p.D + d)) & 0xFFu;
                    qh = __ldg(reinterpret_cast<const uint16_t*>(p.q) + (size_t)bhq * p.D + d);
                    q2[d] = qh | (qh << 16);
                }
                const bool m = p.reference || diff < 8, l = p.reference || diff < 4;
                if (G > 1 && d < p.D) offw[d] = (uint32_t)((m ? 1 : 0) + (l ? 1 : 0)) * SCR_CODE;
                u_mm[r] |= __ballot_sync(0xFFFFFFFFu, m);
                u_lm[r] |= __ballot_sync(0xFFFFFFFFu, l);
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                um[r] = u_mm[r];
                um[8 + r] = u_lm[r];
            }
        }
        __syncwarp();
    };

    const int nrow = (lane % ROW_LANES) >> 1, nhalf = (lane & 1) << 4, ntsub = lane / ROW_LANES;

    // ---- producer: async copies of one stage
    KCursor pk = cursor_at(u_begin);
    int pstage = 0;
    auto issue = [&]() {
        const uint32_t* masks = reinterpret_cast<const uint32_t*>(meta0 + (size_t)pk.slot * META);   // union masks
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
        for (int it = 0; it < TILES / TILES_PER_IT; ++it) {   // nibble planes: only the rows some head reads
            const int t = it * TILES_PER_IT + ntsub;
            if (t < ptiles) {
                const uint32_t dm = nd + t * N_TILE, dl = dm + N_BYTES;
                if (need_m) cp_async16(dm, p.mid4 + pn + t * tile_n);
                else if (G == 1) st_shared_v4(dm, 0x88888888u);              // plane not read: low byte becomes 0x80
                if (need_l) cp_async16(dl, p.last4 + pn + t * tile_n);
                else if (G == 1) st_shared_v4(dl, need_m ? 0x88888888u : 0u);  // low plane not read: low nibble becomes 8
            }
        }
        pstage = (pstage + 1 == STAGES) ? 0 : pstage + 1;
        if (advance(pk) && pk.u < u_end) load_meta(pk.bh, pk.slot);
    };

    // ---- prologue
    load_meta(pk.bh, 0);
    for (int j = 0; j < STAGES - 1; ++j) {
        if (j < total) issue();
        cp_async_commit();
    }

    const int tile = lane >> 3, li = lane & 7;
    // grouped-query scratch: this lane's 8-byte slot of code 0 ("neither plane": low bytes 0x80) never changes
    const uint32_t scr_a = smem_u32(meta0 + NMETA * META) + lane * 8;
    if (G > 1) {
        sts64(scr_a, 0x80808080u, 0x80808080u);
        sts64(scr_a + SCR_ROW, 0x80808080u, 0x80808080u);
    }
    uint32_t acc[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0;
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
        const uint8_t* hm0 = meta0 + (size_t)ck.slot * META + 64;
        const int ch0 = ck.c * KCH;                       // first channel of the stage
        if (G == 1) {
#pragma unroll
            for (int r4 = 0; r4 < KCH / 4; ++r4) {
                const uint4 qv = *reinterpret_cast<const uint4*>(hm0 + (size_t)p.D * 4 + (size_t)(ch0 + r4 * 4) * 4);
#pragma unroll
                for (int rr = 0; rr < 4; ++rr) {
                    // the producer has written the substitutes into the rows it did not fetch
                    const int r = r4 * 4 + rr;
                    const uint2 f = fp[r * 8];
                    const uint32_t M = mp[r * 8], L = lp[r * 8];
                    const uint32_t lbe = (M & 0xF0F0F0F0u) | ((L >> 4) & 0x0F0F0F0Fu);   // low bytes, tokens 0,2,4,6
                    const uint32_t lbo = ((M << 4) & 0xF0F0F0F0u) | (L & 0x0F0F0F0Fu);   // low bytes, tokens 1,3,5,7
                    const uint32_t q2 = rr == 0 ? qv.x : rr == 1 ? qv.y : rr == 2 ? qv.z : qv.w;
                    acc[0][0] = hfma2_bits(__byte_perm(lbe, f.x, 0x6140), q2, acc[0][0]);
                    acc[0][1] = hfma2_bits(__byte_perm(lbo, f.x, 0x7150), q2, acc[0][1]);
                    acc[0][2] = hfma2_bits(__byte_perm(lbe, f.y, 0x6342), q2, acc[0][2]);
                    acc[0][3] = hfma2_bits(__byte_perm(lbo, f.y, 0x7352), q2, acc[0][3]);
                }
            }
        } else {
            // Row r: (a) this lane's low bytes for the codes "mid only" and "both" go to its slots of scratch buffer
            // r & 1 (a plane the union did not fetch leaves garbage there that no head's offset points at), and every
            // head's pair is fetched back through its offset; (b) a row later the pairs are shuffled with the
            // high bytes into k~ words and multiplied.  Only this lane reads what it wrote, so no warp
            // synchronisation is involved; the volatile accesses keep their order.
            const uint32_t hm_a = smem_u32(hm0);
            uint2 fprev = make_uint2(0u, 0u), lbprev[G];
            uint4 ofv[G], qv[G], qprev[G];
#pragma unroll
            for (int r = 0; r <= KCH; ++r) {
                uint2 fcur = make_uint2(0u, 0u), lbcur[G];
#pragma unroll
                for (int g = 0; g < G; ++g) lbcur[g] = make_uint2(0u, 0u);
                if (r < KCH) {
                    if ((r & 3) == 0) {
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            ofv[g] = lds128(hm_a + g * HMETA + (ch0 + r) * 4);
                            qv[g] = lds128(hm_a + g * HMETA + p.D * 4 + (ch0 + r) * 4);
                        }
                    }
                    fcur = fp[r * 8];
                    const uint32_t M = mp[r * 8], L = lp[r * 8];
                    const uint32_t me = M & 0xF0F0F0F0u, mo = (M << 4) & 0xF0F0F0F0u;
                    const uint32_t sb = scr_a + (r & 1) * SCR_ROW;
                    sts64(sb + SCR_CODE, me | 0x08080808u, mo | 0x08080808u);                         // mid only
                    sts64(sb + 2 * SCR_CODE, me | ((L >> 4) & 0x0F0F0F0Fu), mo | (L & 0x0F0F0F0Fu));   // both planes
#pragma unroll
                    for (int g = 0; g < G; ++g) lbcur[g] = lds64(sb + u4w(ofv[g], r & 3));
                }
                if (r > 0) {
                    const int rr = (r - 1) & 3;
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const uint4& qq = rr == 3 ? qprev[g] : qv[g];   // (row 3 of a quad is consumed after the reload)
                        const uint32_t q2 = rr == 0 ? qq.x : rr == 1 ? qq.y : rr == 2 ? qq.z : qq.w;
                        acc[g][0] = hfma2_bits(__byte_perm(lbprev[g].x, fprev.x, 0x6140), q2, acc[g][0]);
                        acc[g][1] = hfma2_bits(__byte_perm(lbprev[g].y, fprev.x, 0x7150), q2, acc[g][1]);
                        acc[g][2] = hfma2_bits(__byte_perm(lbprev[g].x, fprev.y, 0x6342), q2, acc[g][2]);
                        acc[g][3] = hfma2_bits(__byte_perm(lbprev[g].y, fprev.y, 0x7352), q2, acc[g][3]);
                    }
                }
                fprev = fcur;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    lbprev[g] = lbcur[g];
                    if ((r & 3) == 3) qprev[g] = qv[g];
                }
            }
        }
        const long long cbh = ck.bh;
        const int cg = ck.g;
        const bool last_chunk = (ck.c == nch - 1);
        advance(ck);
        if (last_chunk) {  // unit finished: scale, reorder to token order, one 16-byte store per lane and head
            const int blk = cg * TILES + tile;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                if (blk < p.nb) {
                    const uint32_t a0 = hmul2_bits(acc[g][0], p.scale2), a1 = hmul2_bits(acc[g][1], p.scale2);
                    const uint32_t a2 = hmul2_bits(acc[g][2], p.scale2), a3 = hmul2_bits(acc[g][3], p.scale2);
                    uint4 o;
                    o.x = __byte_perm(a0, a1, 0x5410);
                    o.y = __byte_perm(a0, a1, 0x7632);
                    o.z = __byte_perm(a2, a3, 0x5410);
                    o.w = __byte_perm(a2, a3, 0x7632);
                    const size_t row = (size_t)(cbh * G + g) * (size_t)(p.nb + 1) * 64 + (size_t)blk * 64 + li * 8;
                    *reinterpret_cast<uint4*>(p.s + row * 2) = o;
                }
                acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0;
            }
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
                      aligned16(mid4) && aligned16(last4) && aligned16(kq) && aligned16(q) && aligned16(s) &&
                      (group == 1 || group == 2 || group == 4 || group == 8);
    if (!fast) {
        long long total = (long long)bsz * H * group * nb * d_block;
        long long want = (total + 127) / 128;
        int grid = (int)(want < (long long)sm_count() * 16 ? want : (long long)sm_count() * 16);
        count_launch();
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
    const long long units = (long long)p.BH * p.ngroups;
    AKV_REQUIRE(units < (1ll << 30), AKV_ERR_OVERFLOW, "k_cache_compute: too many blocks");
    p.units = (int)units;
    const unsigned short sb = __half_as_ushort(scale);
    p.scale2 = (uint32_t)sb | ((uint32_t)sb << 16);
    p.reference = reference;

    // One CTA per SM.  Pick the channel-chunk size, ring depth and warps per CTA (tunable), trimming the warp
    // count so that every warp gets (nearly) the same whole number of units.
    const int sms = sm_count();
    const int budget = max_dyn_smem();
    // (channels per stage, ring depth): the instantiated combinations; anything else falls back to the default of
    // its group size, and the shared-memory budget below is computed from what is actually launched
    // groups: 8-channel stages (smaller rings, more warps per SM: the consumer does G times the arithmetic per byte)
    const int kch = group > 1 ? (tuning().k_gqa_kch == 16 ? 16 : 8) : tuning().k_kch;
    int stages = tuning().k_stages;
    if (group > 1) stages = kch == 8 ? 4 : 3;
    else if (!((kch == 8 && (stages == 3 || stages == 4 || stages == 6)) || (kch == 16 && stages >= 3 && stages <= 5)))
        stages = (kch == 8) ? 4 : 3;
    const int per_warp = stages * stage_bytes(kch) + nmeta(group) * meta_bytes(D, group) + scratch_bytes(group);
    int wmax = budget / per_warp;
    if (wmax > (group > 1 ? 8 : 16)) wmax = group > 1 ? 8 : 16;   // (the grouped-query kernels are compiled for 256 threads)
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
        // the opt-in shared-memory size is a per-device attribute of the kernel: set it once per (kernel, device) - to
        // the device's maximum, so that every launch shape fits - not on every launch
        static const void* done_kernel[32];
        static int done_device[32];
        static int done_count = 0;                 // (guarded by nothing: a racing thread at worst sets it twice)
        int dev = 0;
        cudaGetDevice(&dev);
        const void* kp = reinterpret_cast<const void*>(kern);
        bool done = false;
        for (int i = 0; i < done_count && i < 32; ++i) done = done || (done_kernel[i] == kp && done_device[i] == dev);
        if (!done) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, budget);
            if (e != cudaSuccess) return cuda_status(e, "k_cache_compute smem attribute");
            if (done_count < 32) {
                done_kernel[done_count] = kp;
                done_device[done_count] = dev;
                ++done_count;
            }
        }
        launch_chained(kern, dim3(grid), dim3(wpc * 32), smem, st, p);
        return AKV_OK;
    };
    int rc;
    if (group == 1) {
        switch (kch * 10 + stages) {
            case 83: rc = go(k_compute_kernel<8, 3, 1>); break;
            case 84: rc = go(k_compute_kernel<8, 4, 1>); break;
            case 86: rc = go(k_compute_kernel<8, 6, 1>); break;
            case 164: rc = go(k_compute_kernel<16, 4, 1>); break;
            case 165: rc = go(k_compute_kernel<16, 5, 1>); break;
            case 163: rc = go(k_compute_kernel<16, 3, 1>); break;
            default:
                set_error("k_cache_compute: no kernel for %d channels x %d stages", kch, stages);
                return AKV_ERR_SHAPE;
        }
    } else if (group == 2) {
        rc = (kch == 8) ? go(k_compute_kernel<8, 4, 2>) : go(k_compute_kernel<16, 3, 2>);
    } else if (group == 4) {
        rc = (kch == 8) ? go(k_compute_kernel<8, 4, 4>) : go(k_compute_kernel<16, 3, 4>);
    } else {
        rc = (kch == 8) ? go(k_compute_kernel<8, 4, 8>) : go(k_compute_kernel<16, 3, 8>);
    }
    if (rc != AKV_OK) return rc;
    return cuda_status(cudaGetLastError(), "k_cache_compute launch");
}

}  // namespace akv
