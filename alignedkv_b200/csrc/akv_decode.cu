// One-call decode step: everything the reference does between receiving (q, k_new, v_new) of one decode token and
// returning the attention output (model/KVCache_AlignedKV.py:116-124), with the wrapper arithmetic of
// extension/k_cache_file.py:97-118,132-159 and extension/v_cache_file.py:97-116,119-190 moved into a handful of
// small kernels around the two streaming kernels:
//   append      residual buffers, per-channel exponent maxima, alignment inputs kq / kqmax
//   (flush)     plane writers, only when the residual buffer reaches 64 tokens
//   q.K^T       akv_k_compute.cu
//   softmax     residual-token scores, -inf padding, fp32 softmax -> fp16 probabilities, and the per-residue-class
//               (token index mod 32) maximum + first position that the magnitude probe needs
//   probe       akv_v_compute.cu, then the threshold byte per (batch, head) with the reference's [B,H,H,D] broadcast
//   P.V         akv_v_compute.cu
//   tail        adds the residual tokens' contribution
#include "akv_exchange.cuh"
#include "akv_save.cuh"

namespace akv {

int launch_v_save(uint8_t*, uint8_t*, uint8_t*, const uint8_t*, int, int, int, int, int, int, int, cudaStream_t);
int launch_k_save(uint8_t*, uint8_t*, uint8_t*, const uint8_t*, int, int, int, int, int, int, int, int,
                  cudaStream_t);
int launch_k_compute(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*,
                     const uint8_t*, uint8_t*, int, int, int, int, int, int, int, float, int, cudaStream_t);
int launch_v_compute(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*,
                     int, int, int, int, int, int, int, int, cudaStream_t);
bool v_compute_takes_probe(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, int, int, int,
                           int);
int launch_v_compute_probe(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*, const uint8_t*,
                           const uint8_t*, uint8_t*, int, int, int, int, int, int, int, int, cudaStream_t);
int launch_v_compute_res(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*, const uint8_t*,
                         const uint8_t*, const uint8_t*, uint8_t*, int, int, int, int, int, int, int, int, cudaStream_t);
bool v_compute_adds_residual(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, int, int, int,
                             int, int, int, int);
int launch_v_split(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*, float*,
                   float*, int, int, int, int, int, int, int, int, cudaStream_t);
int launch_v_split_probe(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*, const uint8_t*,
                         const uint8_t*, uint8_t*, float*, float*, int*, int, int, int, int, int, int, int, int,
                         cudaStream_t);
bool v_split_takes_probe(int, int, int);
long long v_split_scratch_bytes(int, int, int, int);
int launch_v_probe(const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*, int, int, int, int, int, int,
                   cudaStream_t);
int launch_lse_merge(const float*, uint8_t*, int, int, int, cudaStream_t);

constexpr int TOPK = 32;     // residue classes of the magnitude probe (extension/v_cache_file.py:16)
constexpr int SM_CHUNK = 4096;   // scores per CTA of the split softmax
constexpr int BLK = 64;      // tokens per K block (extension/k_cache_file.py:5-6)

// Workspace of one decode step.  H = KV heads, Hq = query heads.
struct Scratch {
    uint16_t* s;         // [B,Hq,R] scores, then probabilities (fp16), R = (nb+1)*64
    uint8_t* kq;         // [B,Hq,D]
    uint8_t* kqmax;      // [B*Hq]
    uint16_t* pval;      // [B,Hq,32]
    int32_t* pidx;       // [B,Hq,32]
    uint16_t* test_o;    // [B,Hq,D]
    uint8_t* amin;       // [B*Hq]
    uint16_t* o_main;    // [B,Hq,D] fp16 result of the exact P.V kernel over the quantized tokens
    float* stats;        // [B*Hq,2] maximum score and sum of exponentials of the softmax
    float* o_main32;     // [B,Hq,D] fp32 result of the order-free P.V kernel
    float* partial;      // chunk partials of the order-free P.V kernel
    float* cstat;        // [B*Hq, chunks, 2] chunk statistics of the split softmax
    uint32_t* cand_val;  // [B*Hq, chunks, 32] residue-class candidates of the split softmax
    int32_t* cand_idx;
};

static size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

static size_t carve(Scratch* sc, uint8_t* base, int B, int H, int G, int D, int max_seq_len, bool order_free) {
    const size_t R = ((size_t)(max_seq_len + BLK - 1) / BLK + 1) * BLK;
    const size_t Q = (size_t)B * H * G;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes); return base ? base + o : nullptr; };
    uint8_t* p;
    p = take(Q * R * 2);        if (sc) sc->s = reinterpret_cast<uint16_t*>(p);
    p = take(Q * D);            if (sc) sc->kq = p;
    p = take(Q);                if (sc) sc->kqmax = p;
    p = take(Q * TOPK * 2);     if (sc) sc->pval = reinterpret_cast<uint16_t*>(p);
    p = take(Q * TOPK * 4);     if (sc) sc->pidx = reinterpret_cast<int32_t*>(p);
    p = take(Q * D * 2);        if (sc) sc->test_o = reinterpret_cast<uint16_t*>(p);
    p = take(Q);                if (sc) sc->amin = p;
    p = take(Q * D * 2);        if (sc) sc->o_main = reinterpret_cast<uint16_t*>(p);
    p = take(Q * 2 * 4);        if (sc) sc->stats = reinterpret_cast<float*>(p);
    const size_t chunks = (R + SM_CHUNK - 1) / SM_CHUNK;
    p = take(Q * chunks * 2 * 4);       if (sc) sc->cstat = reinterpret_cast<float*>(p);
    p = take(Q * chunks * TOPK * 4);    if (sc) sc->cand_val = reinterpret_cast<uint32_t*>(p);
    p = take(Q * chunks * TOPK * 4);    if (sc) sc->cand_idx = reinterpret_cast<int32_t*>(p);
    if (order_free) {
        p = take(Q * D * 4);    if (sc) sc->o_main32 = reinterpret_cast<float*>(p);
        p = take((size_t)v_split_scratch_bytes(B, H, G, max_seq_len));
        if (sc) sc->partial = reinterpret_cast<float*>(p);
    } else if (sc) {
        sc->o_main32 = nullptr;
        sc->partial = nullptr;
    }
    return off;
}

// ------------------------------------------------------------------ append (+ block flush)
// One launch, three roles by block index (128 threads each):
//   [0, BH)            append: residual buffers, per-channel exponent maxima, alignment inputs kq / kqmax of the G
//                      query heads.  With append == 0 nothing is stored (the token belongs to another shard of the
//                      sequence) and only the alignment inputs are built; with append == 2 the token is not stored
//                      either but the exponent maxima take it in (a shard that keeps the maxima of the whole sequence).
//   [BH, 2BH)          (flush only) K block writer: the 63 buffered tokens plus the new one -> planes, block qn/64
//   [2BH, 2BH+BH*D/64) (flush only) V row writer for the same 64 tokens
// The writers take token 63 straight from k_new / v_new, so they do not depend on the append role's stores.
__global__ void __launch_bounds__(128)
append_flush_kernel(uint32_t* __restrict__ restk, uint32_t* __restrict__ restv, uint16_t* __restrict__ k_exp,
                    uint16_t* __restrict__ v_exp, const uint32_t* __restrict__ q, const uint32_t* __restrict__ k_new,
                    const uint32_t* __restrict__ v_new, uint16_t* __restrict__ kq, uint8_t* __restrict__ kqmax,
                    uint8_t* __restrict__ k_first_8, uint8_t* __restrict__ k_mid_4, uint8_t* __restrict__ k_last_4,
                    uint8_t* __restrict__ v_first_8, uint8_t* __restrict__ v_mid_4, uint8_t* __restrict__ v_last_4,
                    int B, int H, int G, int D, int rest_len, int append, int nmb, int max_seq_len, int qn) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ uint32_t red[4];
    pdl_enter();
    const int BH = B * H, hd = D >> 1;
    if ((int)blockIdx.x < BH) {
        const int bh = blockIdx.x, b = bh / H, h = bh - b * H;
        auto exps = [](uint32_t w) { return ((w >> 10) & 0x1Fu) | (((w >> 26) & 0x1Fu) << 8); };  // two exponent bytes
        for (int g = -1; g < G; ++g) {
            // g == -1: store the token and update the maxima; g >= 0: alignment inputs of query head g
            uint32_t m = 0;
            for (int c = threadIdx.x; c < hd; c += blockDim.x) {
                const size_t row = (size_t)bh * hd + c;                              // [B,1,H,D] in words
                if (g < 0) {
                    if (append) {
                        const size_t rrow = (((size_t)b * BLK + rest_len) * H + h) * hd + c;   // [B,64,H,D] in words
                        const uint32_t kw = k_new[row], vw = v_new[row];
                        if (append == 1) {
                            restk[rrow] = kw;
                            restv[rrow] = vw;
                        }
                        // running per-channel maxima of the exponent fields (k_cache_file.py:98-99, v_cache_file.py:98-99)
                        k_exp[row] = (uint16_t)(__vmaxu4(k_exp[row], exps(kw)) & 0xFFFFu);
                        v_exp[row] = (uint16_t)(__vmaxu4(v_exp[row], exps(vw)) & 0xFFFFu);
                    }
                } else {
                    // exponent upper bound of every product q_d * k_{t,d} (k_cache_file.py:136-138); this thread
                    // wrote k_exp[row] itself
                    const size_t qrow = ((size_t)bh * G + g) * hd + c;
                    const uint32_t kq2 = __vadd4(exps(q[qrow]), k_exp[row]) & 0xFFFFu;
                    kq[qrow] = (uint16_t)kq2;
                    m = max(m, max(kq2 & 0xFFu, kq2 >> 8));
                }
            }
            if (g < 0) continue;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            __syncthreads();
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
            __syncthreads();
            if (threadIdx.x == 0) kqmax[(size_t)bh * G + g] = (uint8_t)max(max(red[0], red[1]), max(red[2], red[3]));
        }
        return;
    }
    if ((int)blockIdx.x < 2 * BH) {
        const int bh = blockIdx.x - BH, b = bh / H, h = bh - b * H;
        const uint8_t* rk = reinterpret_cast<const uint8_t*>(restk);
        const uint8_t* kn = reinterpret_cast<const uint8_t*>(k_new);
        auto row = [&](int t) {
            return t < BLK - 1 ? rk + 2 * ((((size_t)b * BLK + t) * H + h) * (size_t)D) : kn + 2 * ((size_t)bh * D);
        };
        k_write_block64(smem, k_first_8, k_mid_4, k_last_4, row, (long long)bh * nmb + qn / BLK, D);
        return;
    }
    {
        const int per_tok = D >> 5, per_bh = BLK * per_tok;              // 32-channel pieces per token / per (b,h)
        const int i = (blockIdx.x - 2 * BH) * blockDim.x + threadIdx.x;   // grid covers BH * per_bh items exactly
        const int bh = i / per_bh, r = i - bh * per_bh, t = r / per_tok, c = r - t * per_tok;
        const int b = bh / H, h = bh - b * H;
        const uint8_t* src = t < BLK - 1
            ? reinterpret_cast<const uint8_t*>(restv) + 2 * ((((size_t)b * BLK + t) * H + h) * (size_t)D + c * 32)
            : reinterpret_cast<const uint8_t*>(v_new) + 2 * ((size_t)bh * D + c * 32);
        const size_t prow = (size_t)bh * max_seq_len + qn + t;
        v_write32_global(reinterpret_cast<const uint4*>(src), v_first_8 + prow * D + c * 32, v_mid_4 + prow * hd + c * 16,
                  v_last_4 + prow * hd + c * 16);
    }
}

// ------------------------------------------------------------------ softmax (+ residual scores, class maxima, probe)
// grid B*Hq, block 256.  Row = [0, qn) aligned scores | [qn, qn+rest) residual scores | -inf up to R.
// CACHED: the row has at most 256*SM_REGS scores and every thread keeps its share in registers, so the row is read
// from memory once instead of three times.  The per-thread and cross-thread summation order is the same either way.
// PROBE (and first8 != nullptr): the magnitude probe (V_cache.cu:104-119; see v_probe_kernel) of this row follows in
// the same CTA from the class maxima it has just found, and lands in test_o.  Both forms pay when the grid is a wave
// or two and the step is bound by the latency of its kernel chain; with many rows the plain form plus a separate
// probe launch keeps more CTAs per SM and is faster.
constexpr int SM_REGS = 32;
constexpr int SM_REGS_512 = 34;   // with 512 threads: rows of up to 17408 scores (16384 cached tokens plus residual blocks)
// Score t of a row as the fp32 softmax sees it: the fp16 score, plus (optional) the additive fp16 mask of its batch
// row, added in fp16 as the reference's in-place `scores += mask` on fp16 tensors does (model/KVCache_AlignedKV.py:119-120).
__device__ __forceinline__ float masked_score(const uint16_t* __restrict__ row, const __half* __restrict__ mrow, int t) {
    __half s = __ushort_as_half(row[t]);
    if (mrow) s = __hadd(s, mrow[t]);
    return __half2float(s);
}
// Scores of the residual tokens of one (batch, query head) row, by a CTA of 256 threads: thread = (token tid / 4,
// quarter tid % 4 of the channels in 16-byte pieces), all loads of a row in flight at once, fp32 dot product rounded to
// fp16, then divided by sqrt(D) and rounded again, which is what `matmul(q, restk^T) / sqrt(D)` on fp16 tensors
// produces (k_cache_file.py:156-157).  Only tokens with t_lo <= qn + r < t_hi are written (a row split across CTAs).
__device__ __forceinline__ void residual_scores(uint16_t* __restrict__ row, const __half* __restrict__ qr,
                                                const __half* __restrict__ restk, int b, int h, int H, int D, int qn,
                                                int rest, float sqrt_d, int t_lo, int t_hi) {
    const int tid = threadIdx.x;
    for (int r0 = 0; r0 < rest; r0 += 64) {       // (the residual buffer holds at most 64 tokens: one round)
        const int r = r0 + (tid >> 2), c = tid & 3;
        const bool mine = r < rest && qn + r >= t_lo && qn + r < t_hi;
        float acc = 0.f;
        if (mine) {
            const __half* kr = restk + (((size_t)b * BLK + r) * H + h) * D;
            for (int d = c * 8; d < D; d += 32) {
                const uint4 kv = *reinterpret_cast<const uint4*>(kr + d), qv = *reinterpret_cast<const uint4*>(qr + d);
                const __half2* k2 = reinterpret_cast<const __half2*>(&kv);
                const __half2* q2 = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 kf = __half22float2(k2[i]), qf = __half22float2(q2[i]);
                    acc = fmaf(qf.x, kf.x, acc);
                    acc = fmaf(qf.y, kf.y, acc);
                }
            }
        }
        acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
        acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 2);
        if (mine && c == 0) row[qn + r] = __half_as_ushort(__float2half_rn(__half2float(__float2half_rn(acc)) / sqrt_d));
    }
}

// NT threads per CTA (256, or 512 for rows of up to 512*SM_REGS scores that one CTA keeps in registers).
// RG: scores a thread keeps in registers (CACHED): SM_REGS, or fewer for short rows - with 17 (rows of up to 4352
// scores) two CTAs of 256 threads fit an SM instead of one, and 256 rows run as one wave.
template <bool CACHED, bool PROBE, int NT, int RG = (NT == 512 ? SM_REGS_512 : SM_REGS)>
__global__ void __launch_bounds__(NT, (RG <= 17 && NT == 256) ? 2 : 0)
softmax_kernel(uint16_t* __restrict__ s, const __half* __restrict__ q, const __half* __restrict__ restk,
               uint16_t* __restrict__ pval, int32_t* __restrict__ pidx, float* __restrict__ stats,
               const uint8_t* __restrict__ first8, uint16_t* __restrict__ test_o, int max_seq_len, int H, int G, int D,
               int R, int qn, int rest, float sqrt_d, const __half* __restrict__ mask, long long mask_stride,
               const __half* __restrict__ restv, uint16_t* __restrict__ res) {
    constexpr int NW = NT / 32;
    constexpr int REGS = RG;                                     // scores a thread keeps (CACHED)
    __shared__ float redf[NW];
    __shared__ uint32_t cand_v[NT];
    __shared__ int32_t cand_i[NT];
    pdl_enter();
    const int bhq = blockIdx.x, Hq = H * G, b = bhq / Hq, h = (bhq - b * Hq) / G;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint16_t* row = s + (size_t)bhq * R;
    const __half* mrow = mask ? mask + (size_t)b * mask_stride : nullptr;
    const int len = qn + rest;
    residual_scores(row, q + (size_t)bhq * D, restk, b, h, H, D, qn, rest, sqrt_d, 0, len);
    __syncthreads();
    float x[CACHED ? REGS : 1];
    // pass 1: maximum
    float m = -INFINITY;
    if (CACHED) {
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int t = tid + NT * i;
            x[i] = t < len ? masked_score(row, mrow, t) : -INFINITY;
            m = fmaxf(m, x[i]);
        }
    } else {
        for (int t = tid; t < len; t += NT) m = fmaxf(m, masked_score(row, mrow, t));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane == 0) redf[warp] = m;
    __syncthreads();
    m = redf[0];
#pragma unroll
    for (int w = 1; w < NW; ++w) m = fmaxf(m, redf[w]);
    __syncthreads();
    // pass 2: sum of exponentials (fp32, as F.softmax(scores.float()) does; model/KVCache_AlignedKV.py:121)
    float sum = 0.f;
    if (CACHED) {
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            if (tid + NT * i < len) {
                x[i] = expf(x[i] - m);
                sum += x[i];
            }
        }
    } else {
        for (int t = tid; t < len; t += NT) sum += expf(masked_score(row, mrow, t) - m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (lane == 0) redf[warp] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) sum += redf[w];
    if (tid == 0) {
        stats[(size_t)bhq * 2] = m;
        stats[(size_t)bhq * 2 + 1] = sum;
    }
    // pass 3: probabilities, and this thread's residue class (tid % 32): largest probability over the quantized
    // tokens with its first position (torch.max over the group axis keeps the first maximum; v_cache_file.py:128-130)
    uint32_t best = 0;
    int32_t best_g = 0;
    if (CACHED) {
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int t = tid + NT * i;
            if (t < R) {
                uint16_t pb = 0;   // exp(-inf - m) = 0
                if (t < len) pb = __half_as_ushort(__float2half_rn(x[i] / sum));
                row[t] = pb;
                if (t < qn && pb > best) {   // probabilities are non-negative: bit patterns order like values
                    best = pb;
                    best_g = t >> 5;
                }
            }
        }
    } else {
        for (int t = tid; t < R; t += NT) {
            uint16_t pb = 0;
            if (t < len) pb = __half_as_ushort(__float2half_rn(expf(masked_score(row, mrow, t) - m) / sum));
            row[t] = pb;
            if (t < qn && pb > best) {
                best = pb;
                best_g = t >> 5;
            }
        }
    }
    cand_v[tid] = best;
    cand_i[tid] = best_g;
    __syncthreads();
    if (tid < TOPK) {
        uint32_t bv = cand_v[tid];
        int32_t bi = cand_i[tid];
        for (int w = 1; w < NW; ++w) {
            const uint32_t v = cand_v[tid + 32 * w];
            const int32_t i = cand_i[tid + 32 * w];
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        pval[(size_t)bhq * TOPK + tid] = (uint16_t)bv;
        pidx[(size_t)bhq * TOPK + tid] = bi;
        if (PROBE) {
            cand_v[tid] = bv;
            cand_i[tid] = bi;
        }
    }
    if (!PROBE || first8 == nullptr || qn == 0) return;   // (uniform)
    __syncthreads();
    // probe: o_test[d] = sum_j |half((first_8[row_j][d] << 8) + 0x80)| * p_j over the class maxima, rows
    // row_j = class position * 32 + j, accumulated in fp16 in j order; all row gathers go out before the chain starts
    const uint8_t* F = first8 + (size_t)(bhq / G) * max_seq_len * D;
    for (int c = tid; c < (D >> 1); c += NT) {
        uint32_t f[TOPK];
#pragma unroll
        for (int j = 0; j < TOPK; ++j) {
            long long r = (long long)cand_i[j] * TOPK + j;
            r = r >= max_seq_len ? max_seq_len - 1 : r;
            f[j] = __ldg(reinterpret_cast<const uint16_t*>(F + (size_t)r * D + 2 * c));
        }
        uint32_t acc = 0;
#pragma unroll
        for (int j = 0; j < TOPK; ++j) {
            const uint32_t v = __byte_perm(f[j], 0x80u, 0x1404) & 0x7FFF7FFFu;
            acc = hfma2_bits(v, cand_v[j] | (cand_v[j] << 16), acc);
        }
        reinterpret_cast<uint32_t*>(test_o)[(size_t)bhq * (D >> 1) + c] = acc;
    }
    if (res == nullptr || rest <= 0) return;              // (uniform)
    // The residual tokens' part of the output, half(sum_r p[qn + r] * restv[r]) (extension/v_cache_file.py:189), for the
    // P.V kernel to add in its epilogue - computed here by the threads the probe leaves idle (it occupies D/2 of them),
    // so that no tail launch is needed.  Item = (channel pair, third of the tokens); fp32 sums, added in a fixed order.
    __shared__ float part[3][256];
    {
        const int hd = D >> 1, idle0 = hd < NT ? hd : 0, nidle = NT - idle0;
        if (tid >= idle0) {
            for (int i = tid - idle0; i < 3 * hd; i += nidle) {
                const int g = i / hd, c = i - g * hd;
                const __half* vr = restv + ((size_t)b * BLK * H + h) * D + 2 * c;
                const size_t vs = (size_t)H * D;
                float pv[22];
                __half2 vv[22];
#pragma unroll
                for (int j = 0; j < 22; ++j) {
                    const int r = g + 3 * j;
                    const bool on = r < rest;
                    pv[j] = on ? __half2float(__ushort_as_half(row[qn + r])) : 0.f;
                    vv[j] = on ? *reinterpret_cast<const __half2*>(vr + (size_t)r * vs) : __half2(__half(0.f), __half(0.f));
                }
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int j = 0; j < 22; ++j) {
                    const float2 f = __half22float2(vv[j]);
                    a0 = fmaf(pv[j], f.x, a0);
                    a1 = fmaf(pv[j], f.y, a1);
                }
                part[g][2 * c] = a0;
                part[g][2 * c + 1] = a1;
            }
        }
    }
    __syncthreads();
    for (int d = tid; d < D; d += NT)
        res[(size_t)bhq * D + d] = __half_as_ushort(__float2half_rn((part[0][d] + part[1][d]) + part[2][d]));
}

// ------------------------------------------------------------------ softmax over long rows, split across CTAs
// With few (batch, head) rows and a long sequence one CTA per row cannot keep up, so the row is cut into chunks of
// SM_CHUNK scores: (1) per chunk the maximum and the sum of exponentials relative to it (the chunk that holds the
// residual tokens computes their scores first), (2) every chunk CTA combines the chunk statistics into the row's
// (max, sum), writes its probabilities and its candidates for the 32 residue classes, (3) one small CTA per row
// reduces the candidates (largest probability, then first position) and stores the row statistics.
__global__ void __launch_bounds__(256)
softmax_chunk_stats_kernel(uint16_t* __restrict__ s, const __half* __restrict__ q, const __half* __restrict__ restk,
                           float* __restrict__ cstat, int H, int G, int D, int R, int qn, int rest, float sqrt_d,
                           int chunks, const __half* __restrict__ mask, long long mask_stride) {
    __shared__ float redf[8];
    const int bhq = blockIdx.y, ch = blockIdx.x, Hq = H * G, b = bhq / Hq, h = (bhq - b * Hq) / G;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint16_t* row = s + (size_t)bhq * R;
    const __half* mrow = mask ? mask + (size_t)b * mask_stride : nullptr;
    const int len = qn + rest;
    const int t0 = ch * SM_CHUNK, t1 = min(len, t0 + SM_CHUNK);
    // residual-token scores by the chunk(s) that hold them
    residual_scores(row, q + (size_t)bhq * D, restk, b, h, H, D, qn, rest, sqrt_d, t0, t1);
    __syncthreads();
    float m = -INFINITY;
    for (int t = t0 + tid; t < t1; t += 256) m = fmaxf(m, masked_score(row, mrow, t));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane == 0) redf[warp] = m;
    __syncthreads();
    m = redf[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, redf[w]);
    __syncthreads();
    float sum = 0.f;
    for (int t = t0 + tid; t < t1; t += 256) sum += expf(masked_score(row, mrow, t) - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (lane == 0) redf[warp] = sum;
    __syncthreads();
    if (tid == 0) {
        sum = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) sum += redf[w];
        cstat[((size_t)bhq * chunks + ch) * 2] = m;            // -inf for an empty chunk
        cstat[((size_t)bhq * chunks + ch) * 2 + 1] = sum;
    }
}

__global__ void __launch_bounds__(256)
softmax_chunk_write_kernel(uint16_t* __restrict__ s, const float* __restrict__ cstat, uint32_t* __restrict__ cand_val,
                           int32_t* __restrict__ cand_idx, int R, int qn, int len, int chunks, int stat_chunks,
                           int stat_ranks, int t_base, const __half* __restrict__ mask, long long mask_stride, int Hq) {
    // chunks: row stride (in chunks) of the candidate arrays, at least the chunks of this row held here (the grid);
    // stat_chunks: chunks whose statistics make up the row's (they include the other shards' when the sequence is
    // sharded), laid out as stat_ranks blocks of [rows][stat_chunks / stat_ranks] as an all-gather leaves them;
    // t_base: position of local token 0 in the whole sequence (a multiple of 32, so residue classes are the same
    // locally and globally)
    const int spr = stat_chunks / stat_ranks;       // chunks per rank block
    auto stat = [&](int c) {
        const int r = c / spr;
        return cstat + (((size_t)r * gridDim.y + blockIdx.y) * spr + (c - r * spr)) * 2;
    };
    __shared__ uint32_t cand_v[256];
    __shared__ int32_t cand_i[256];
    __shared__ float term[256];
    __shared__ float wmax[8];
    const int bhq = blockIdx.y, ch = blockIdx.x, tid = threadIdx.x;
    uint16_t* row = s + (size_t)bhq * R;
    const __half* mrow = mask ? mask + (size_t)(bhq / Hq) * mask_stride : nullptr;
    // Row statistics from the chunk statistics (every CTA of the row computes the same values): the maximum, then the
    // sum of l_c exp(m_c - m) added IN CHUNK ORDER.  The loads and the exponentials of up to 256 chunks are done in
    // parallel, one per thread; only the additions are serial, out of shared memory - the same operations in the same
    // order as a loop over the chunks, at a fraction of its latency (an empty chunk contributes an exact 0).
    float m = -INFINITY;
    for (int c0 = 0; c0 < stat_chunks; c0 += 256) {
        float v = c0 + tid < stat_chunks ? stat(c0 + tid)[0] : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
        if ((tid & 31) == 0) wmax[tid >> 5] = v;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < 8; ++w) m = fmaxf(m, wmax[w]);
        __syncthreads();
    }
    float sum = 0.f;
    for (int c0 = 0; c0 < stat_chunks; c0 += 256) {
        float tm = 0.f;
        if (c0 + tid < stat_chunks) {
            const float* st2 = stat(c0 + tid);
            const float mc = st2[0];
            if (mc > -INFINITY) tm = st2[1] * expf(mc - m);
        }
        term[tid] = tm;
        __syncthreads();
        const int cnt = min(256, stat_chunks - c0);
        for (int c = 0; c < cnt; ++c) sum += term[c];
        __syncthreads();
    }
    const int t0 = ch * SM_CHUNK, t1 = min(R, t0 + SM_CHUNK);
    uint32_t best = 0;
    int32_t best_g = 0;
    for (int t = t0 + tid; t < t1; t += 256) {     // (t0 and 256 are multiples of 32: a thread keeps its class)
        uint16_t pb = 0;
        if (t < len) pb = __half_as_ushort(__float2half_rn(expf(masked_score(row, mrow, t) - m) / sum));
        row[t] = pb;
        if (t < qn && pb > best) {
            best = pb;
            best_g = (t_base + t) >> 5;
        }
    }
    cand_v[tid] = best;
    cand_i[tid] = best_g;
    __syncthreads();
    if (tid < TOPK) {
        uint32_t bv = cand_v[tid];
        int32_t bi = cand_i[tid];
        for (int w = 1; w < 8; ++w) {
            const uint32_t v = cand_v[tid + 32 * w];
            const int32_t i = cand_i[tid + 32 * w];
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        cand_val[((size_t)bhq * chunks + ch) * TOPK + tid] = bv;
        cand_idx[((size_t)bhq * chunks + ch) * TOPK + tid] = bi;
    }
}

__global__ void __launch_bounds__(32)
softmax_class_reduce_kernel(const float* __restrict__ cstat, const uint32_t* __restrict__ cand_val,
                            const int32_t* __restrict__ cand_idx, uint16_t* __restrict__ pval,
                            int32_t* __restrict__ pidx, float* __restrict__ stats, int chunks, int ranks) {
    // ranks == 1: cand_val / cand_idx are [rows][chunks][32].  ranks > 1 (gathered from the shards of a sequence):
    // cand_val points at `ranks` blocks of {values [rows][chunks/ranks][32], positions [rows][chunks/ranks][32]} and
    // cand_idx is unused.
    const int bhq = blockIdx.x, tid = threadIdx.x;
    const int cpr = chunks / ranks;
    const size_t block = (size_t)gridDim.x * cpr * TOPK;          // one array of one rank
    auto val_at = [&](int c) -> const uint32_t* {
        const int r = c / cpr;
        const size_t e = ((size_t)bhq * cpr + (c - r * cpr)) * TOPK + tid;
        return ranks == 1 ? cand_val + e : cand_val + (size_t)r * 2 * block + e;
    };
    // chunks are in position order: a later chunk wins only when larger.  Eight chunks' values are loaded at a time;
    // the position is fetched for the winner only.
    uint32_t bv = 0;
    int bc = -1;
    for (int c0 = 0; c0 < chunks; c0 += 8) {
        uint32_t v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = c0 + j < chunks ? *val_at(c0 + j) : 0u;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (v[j] > bv) { bv = v[j]; bc = c0 + j; }
    }
    int32_t bi = 0;
    if (bc >= 0) {
        const int r = bc / cpr;
        const size_t e = ((size_t)bhq * cpr + (bc - r * cpr)) * TOPK + tid;
        bi = ranks == 1 ? cand_idx[e] : reinterpret_cast<const int32_t*>(cand_val)[(size_t)r * 2 * block + block + e];
    }
    pval[(size_t)bhq * TOPK + tid] = (uint16_t)bv;
    pidx[(size_t)bhq * TOPK + tid] = bi;
    if (cstat != nullptr) {
        // row statistics: maximum, then the sum of l_c exp(m_c - m) in chunk order; lane = chunk, 32 at a time, the
        // additions serial through shuffles (the same operations in the same order as a loop over the chunks)
        const float* cs = cstat + (size_t)bhq * chunks * 2;
        float m = -INFINITY;
        for (int c0 = 0; c0 < chunks; c0 += 32) {
            float v = c0 + tid < chunks ? cs[(size_t)(c0 + tid) * 2] : -INFINITY;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
            m = fmaxf(m, v);
        }
        float sum = 0.f;
        for (int c0 = 0; c0 < chunks; c0 += 32) {
            float tm = 0.f;
            if (c0 + tid < chunks) {
                const float mc = cs[(size_t)(c0 + tid) * 2];
                if (mc > -INFINITY) tm = cs[(size_t)(c0 + tid) * 2 + 1] * expf(mc - m);
            }
            const int cnt = min(32, chunks - c0);
            for (int c = 0; c < cnt; ++c) sum += __shfl_sync(0xFFFFFFFFu, tm, c);
        }
        if (tid == 0) {
            stats[(size_t)bhq * 2] = m;
            stats[(size_t)bhq * 2 + 1] = sum;
        }
    }
}

// ------------------------------------------------------------------ threshold byte per (batch, query head)
// One warp per row (v_threshold_warp).  Used when the P.V kernel that follows does not compute the byte itself.
__global__ void __launch_bounds__(128)
amin_kernel(const uint16_t* __restrict__ test_o, const uint8_t* __restrict__ v_exp, uint8_t* __restrict__ amin,
            int BHq, int H, int G, int D) {
    pdl_enter();
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= BHq) return;
    const int lane = threadIdx.x & 31;
    const uint32_t m = v_threshold_warp(test_o, v_exp, i, H, G, D, lane);
    if (lane == 0) amin[i] = (uint8_t)m;
}

// ------------------------------------------------------------------ tail: residual tokens of P.V, final outputs
// out = half(o_main + half(sum_r p[qn+r] * restv[r])) (v_cache_file.py:189); grid B*Hq.  With an fp32 main result
// (order-free P.V) the residual sum is added in fp32 and rounded once.  packed (optional): one row
// (max score, sum of exponentials, output[0..D-1]) in fp32 per (batch, query head), the record ranks exchange when
// the sequence is sharded.  x.R > 0: the CTA then exchanges its record with the other ranks through peer memory and
// writes the merged row (x.out).
__global__ void __launch_bounds__(256)
tail_kernel(const uint16_t* __restrict__ o_main, const float* __restrict__ o_main32, const uint16_t* __restrict__ p,
            const __half* __restrict__ restv, __half* __restrict__ out, const float* __restrict__ stats,
            float* __restrict__ packed, int H, int G, int D, int R, int qn, int rest, int chunks, const XchgParams x) {
    pdl_enter();
    const int bhq = blockIdx.x, Hq = H * G, b = bhq / Hq, h = (bhq - b * Hq) / G;
    // residual sum: item = (channel pair, quarter g of the tokens: r = g, g+4, ...), all of an item's loads in flight
    // at once; the four partial sums of a channel are added in order g = 0..3
    __shared__ float part[4][1024];
    const int hd = D >> 1;
    if (rest > 0) {
        const uint16_t* pr = p + (size_t)bhq * R + qn;
        const size_t vs = (size_t)H * D;
        for (int i = threadIdx.x; i < 4 * hd; i += blockDim.x) {
            const int g = i / hd, c = i - g * hd;
            const __half* vr = restv + ((size_t)b * BLK * H + h) * D + 2 * c;
            float pv[16];
            __half2 vv[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int r = g + 4 * j;
                const bool on = r < rest;
                pv[j] = on ? __half2float(__ushort_as_half(pr[r])) : 0.f;
                vv[j] = on ? *reinterpret_cast<const __half2*>(vr + (size_t)r * vs) : __half2(__half(0.f), __half(0.f));
            }
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float2 f = __half22float2(vv[j]);
                a0 = fmaf(pv[j], f.x, a0);
                a1 = fmaf(pv[j], f.y, a1);
            }
            part[g][2 * c] = a0;
            part[g][2 * c + 1] = a1;
        }
        __syncthreads();
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float acc = rest > 0 ? ((part[0][d] + part[1][d]) + part[2][d]) + part[3][d] : 0.f;
        float v;
        if (o_main32 && chunks > 0) {
            // o_main32 holds the order-free kernel's chunk partials [chunks][D] of this row: added in chunk order
            float m = 0.f;
            for (int c = 0; c < chunks; ++c) m += o_main32[((size_t)bhq * chunks + c) * D + d];
            v = m + acc;
        } else if (o_main32) v = o_main32[(size_t)bhq * D + d] + acc;
        else v = (o_main ? __half2float(__ushort_as_half(o_main[(size_t)bhq * D + d])) : 0.f) +
                 __half2float(__float2half_rn(acc));
        if (out) out[(size_t)bhq * D + d] = __float2half_rn(v);
        if (packed) packed[(size_t)bhq * (D + 2) + 2 + d] = o_main32 ? v : __half2float(__float2half_rn(v));
    }
    if (packed && threadIdx.x == 0) {
        packed[(size_t)bhq * (D + 2)] = stats[(size_t)bhq * 2];
        packed[(size_t)bhq * (D + 2) + 1] = stats[(size_t)bhq * 2 + 1];
    }
    if (x.R > 0) {
        // sequence shards: the row's record goes to every rank and the merged row comes back (akv_exchange.cuh)
        // (the residual sums' scratch is free by now and holds the collected records)
        static_assert(XCHG_ROW_FLOATS <= 4 * 1024, "the collected row has to fit the residual scratch");
        __shared__ uint8_t* s_buf[XCHG_MAX_RANKS];
        __syncthreads();
        exchange_merge_row(x, packed + (size_t)bhq * (D + 2), bhq, s_buf, &part[0][0]);
    }
}

// ------------------------------------------------------------------ magnitude probe across sequence shards
// The 32 winning tokens of a row can lie on any shard.  Each shard writes the high-byte rows of the winners it holds
// (zeros for the others) - rows[bhq][j][0..D) for token pidx[bhq][j]*32 + j of the whole sequence - the shards' buffers
// are added up, and every shard then runs the same fp16 chain over the same bytes (V_cache.cu:104-119).
__global__ void __launch_bounds__(128)
probe_rows_gather_kernel(const uint8_t* __restrict__ first8, const int32_t* __restrict__ pidx, uint8_t* __restrict__ rows,
                         int G, int D, int max_seq_len, int qn, int t_base) {
    const long long bhq = blockIdx.x;
    const uint8_t* F = first8 + (size_t)(bhq / G) * max_seq_len * D;
    const int wpr = D >> 2;                                  // 32-bit words per row
    for (int i = threadIdx.x; i < TOPK * wpr; i += blockDim.x) {
        const int j = i / wpr, w = i - j * wpr;
        const long long local = (long long)pidx[bhq * TOPK + j] * TOPK + j - t_base;
        uint32_t v = 0;
        if (local >= 0 && local < qn) v = reinterpret_cast<const uint32_t*>(F + (size_t)local * D)[w];
        reinterpret_cast<uint32_t*>(rows + ((size_t)bhq * TOPK + j) * D)[w] = v;
    }
}

__global__ void __launch_bounds__(128)
probe_from_rows_kernel(const uint8_t* __restrict__ rows, const uint16_t* __restrict__ pval, uint16_t* __restrict__ test_o,
                       int D) {
    const long long bhq = blockIdx.x;
    for (int c = threadIdx.x; c < (D >> 1); c += blockDim.x) {
        uint32_t acc = 0;
#pragma unroll 8
        for (int j = 0; j < TOPK; ++j) {
            const uint32_t f = reinterpret_cast<const uint16_t*>(rows + ((size_t)bhq * TOPK + j) * D)[c];
            const uint32_t sv = pval[bhq * TOPK + j];
            acc = hfma2_bits(__byte_perm(f, 0x80u, 0x1404) & 0x7FFF7FFFu, sv | (sv << 16), acc);
        }
        reinterpret_cast<uint32_t*>(test_o)[(size_t)bhq * (D >> 1) + c] = acc;
    }
}

// ------------------------------------------------------------------ rollback of appended tokens
// Undo appends: the exponent maxima are put back from copies the caller took earlier, and the K nibble planes of
// blocks that were written since are cleared (the K writer ADDS nibbles, extension/csrc/K_cache.cu:52-56, so a block
// has to be zero before it is written again).  High bytes, V planes and residual rows need nothing: they are
// overwritten by plain stores when the positions are appended again.  grid B*H, 128 threads.
__global__ void __launch_bounds__(128)
rollback_kernel(uint4* __restrict__ k_mid_4, uint4* __restrict__ k_last_4, uint4* __restrict__ k_exp,
                uint4* __restrict__ v_exp, const uint4* __restrict__ k_exp_saved, const uint4* __restrict__ v_exp_saved,
                int D, int nmb, int first_block, int n_blocks) {
    pdl_enter();
    const long long bh = blockIdx.x;
    const int vec_per_block = D * (BLK / 2) / 16;                     // 16-byte pieces of one nibble-plane block
    uint4* m = k_mid_4 + (bh * nmb + first_block) * vec_per_block;
    uint4* l = k_last_4 + (bh * nmb + first_block) * vec_per_block;
    for (int i = threadIdx.x; i < n_blocks * vec_per_block; i += blockDim.x) {
        m[i] = make_uint4(0, 0, 0, 0);
        l[i] = make_uint4(0, 0, 0, 0);
    }
    for (int i = threadIdx.x; i < D / 16; i += blockDim.x) {
        k_exp[bh * (D / 16) + i] = k_exp_saved[bh * (D / 16) + i];
        v_exp[bh * (D / 16) + i] = v_exp_saved[bh * (D / 16) + i];
    }
}

// ------------------------------------------------------------------ optional per-kernel timing
struct Timing {
    static constexpr int CAP = 4096;
    cudaEvent_t ev[CAP][4];
    int created = 0, used = 0;
};
static Timing g_timing;
static cudaEvent_t* g_shard_timing = nullptr;   // slot of the sharded step in progress (akv_shard_step)
static thread_local bool g_timing_off = false;  // set around a step that must not create events (allocation-free entry)

static cudaEvent_t* timing_slot() {
    if (!tuning().timing || g_timing_off) return nullptr;
    Timing& t = g_timing;
    if (t.used >= Timing::CAP) return nullptr;
    if (t.used >= t.created) {
        for (int i = 0; i < 4; ++i)
            if (cudaEventCreate(&t.ev[t.created][i]) != cudaSuccess) return nullptr;
        ++t.created;
    }
    return t.ev[t.used++];
}

}  // namespace akv

using namespace akv;

extern "C" {

long long akv_decode_scratch_bytes_ex(int bsz, int n_kv_heads, int group, int head_dim, int max_seq_len, int flags) {
    if (bsz <= 0 || n_kv_heads <= 0 || group <= 0 || head_dim <= 0 || max_seq_len <= 0) return -1;
    return (long long)carve(nullptr, nullptr, bsz, n_kv_heads, group, head_dim, max_seq_len,
                            (flags & AKV_STEP_ORDER_FREE) != 0);
}

long long akv_decode_scratch_bytes(int bsz, int n_heads, int head_dim, int max_seq_len) {
    return akv_decode_scratch_bytes_ex(bsz, n_heads, 1, head_dim, max_seq_len, 0);
}

int akv_timing_reset(void) {
    g_timing.used = 0;
    return AKV_OK;
}

// Median duration (microseconds) of the q.K^T and P.V launches recorded since the last reset (the median, so that a
// step that was held up by something else on the machine does not move the figure); the caller must have
// synchronised the stream.  Returns the number of recorded steps.
int akv_timing_read(double* k_us, double* v_us) {
    static float ks[Timing::CAP], vs[Timing::CAP];
    int n = 0;
    for (int i = 0; i < g_timing.used; ++i) {
        float a = 0, b = 0;
        if (cudaEventElapsedTime(&a, g_timing.ev[i][0], g_timing.ev[i][1]) != cudaSuccess) continue;
        if (cudaEventElapsedTime(&b, g_timing.ev[i][2], g_timing.ev[i][3]) != cudaSuccess) continue;
        ks[n] = a * 1e3f;
        vs[n] = b * 1e3f;
        ++n;
    }
    auto median = [](float* x, int m) -> double {
        if (m == 0) return 0.0;
        for (int i = 1; i < m; ++i) {   // insertion sort: at most a few thousand entries, off the hot path
            float v = x[i];
            int j = i - 1;
            for (; j >= 0 && x[j] > v; --j) x[j + 1] = x[j];
            x[j + 1] = v;
        }
        return (m & 1) ? x[m / 2] : 0.5 * (x[m / 2 - 1] + x[m / 2]);
    };
    if (k_us) *k_us = median(ks, n);
    if (v_us) *v_us = median(vs, n);
    return n;
}

int akv_decode_step_ex(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                       void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q, const void* k_new,
                       const void* v_new, void* out, void* packed_out, void* scratch, long long scratch_bytes, int bsz,
                       int n_kv_heads, int group, int head_dim, int max_seq_len, int rest_len, int rest_start,
                       int flags, void* stream) {
    return akv_decode_step_masked(k_first_8, k_mid_4, k_last_4, v_first_8, v_mid_4, v_last_4, k_exp_max, v_exp_max, restk,
                                  restv, q, k_new, v_new, out, packed_out, nullptr, 0, scratch, scratch_bytes, bsz,
                                  n_kv_heads, group, head_dim, max_seq_len, rest_len, rest_start, flags, stream);
}

static int decode_step_impl(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                            void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q, const void* k_new,
                            const void* v_new, void* out, void* packed_out, const void* mask, long long mask_stride,
                            void* scratch, long long scratch_bytes, int bsz, int n_kv_heads, int group, int head_dim,
                            int max_seq_len, int rest_len, int rest_start, int flags, void* stream, const XchgParams& xp);

int akv_decode_step_masked(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                           void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q, const void* k_new,
                           const void* v_new, void* out, void* packed_out, const void* mask, long long mask_stride,
                           void* scratch, long long scratch_bytes, int bsz, int n_kv_heads, int group, int head_dim,
                           int max_seq_len, int rest_len, int rest_start, int flags, void* stream) {
    set_error("");
    return decode_step_impl(k_first_8, k_mid_4, k_last_4, v_first_8, v_mid_4, v_last_4, k_exp_max, v_exp_max, restk, restv,
                            q, k_new, v_new, out, packed_out, mask, mask_stride, scratch, scratch_bytes, bsz, n_kv_heads,
                            group, head_dim, max_seq_len, rest_len, rest_start, flags, stream, XchgParams{});
}

int akv_decode_step_exchange(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4,
                             void* v_last_4, void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q,
                             const void* k_new, const void* v_new, void* merged_out, void* packed_out, void* scratch,
                             long long scratch_bytes, int bsz, int n_kv_heads, int group, int head_dim, int max_seq_len,
                             int rest_len, int rest_start, int flags, void* const* bufs, int rank, int n_ranks,
                             unsigned int epoch, int timeout_ms, void* stream) {
    set_error("");
    AKV_REQUIRE(packed_out && merged_out, AKV_ERR_NULL, "decode_step_exchange: null pointer");
    AKV_REQUIRE(bsz > 0 && n_kv_heads > 0 && group > 0, AKV_ERR_SHAPE, "decode_step_exchange: bad extent");
    XchgParams xp;
    const int rc = fill_exchange(&xp, bufs, rank, n_ranks, merged_out, bsz * n_kv_heads * group, head_dim, epoch,
                                 timeout_ms);
    if (rc != AKV_OK) return rc;
    return decode_step_impl(k_first_8, k_mid_4, k_last_4, v_first_8, v_mid_4, v_last_4, k_exp_max, v_exp_max, restk, restv,
                            q, k_new, v_new, nullptr, packed_out, nullptr, 0, scratch, scratch_bytes, bsz, n_kv_heads,
                            group, head_dim, max_seq_len, rest_len, rest_start, flags, stream, xp);
}

static int decode_step_impl(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                            void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q, const void* k_new,
                            const void* v_new, void* out, void* packed_out, const void* mask, long long mask_stride,
                            void* scratch, long long scratch_bytes, int bsz, int n_kv_heads, int group, int head_dim,
                            int max_seq_len, int rest_len, int rest_start, int flags, void* stream, const XchgParams& xp) {
    AKV_REQUIRE(!mask || ((reinterpret_cast<uintptr_t>(mask) & 1u) == 0 && mask_stride >= 0), AKV_ERR_ALIGN,
                "decode_step: the mask must be 2-byte aligned with a non-negative row stride");
    const __half* mk = static_cast<const __half*>(mask);
    const int B = bsz, H = n_kv_heads, G = group, D = head_dim;
    const bool reference = (flags & AKV_STEP_REFERENCE) != 0, order_free = (flags & AKV_STEP_ORDER_FREE) != 0;
    const bool append = (flags & AKV_STEP_NO_APPEND) == 0;
    AKV_REQUIRE(k_first_8 && k_mid_4 && k_last_4 && v_first_8 && v_mid_4 && v_last_4 && k_exp_max && v_exp_max &&
                restk && restv && q && (out || packed_out) && scratch && (!append || (k_new && v_new)), AKV_ERR_NULL,
                "decode_step: null pointer");
    AKV_REQUIRE(B > 0 && H > 0 && G > 0 && G <= 64 && D > 0 && D % 64 == 0 && D <= 1024 && max_seq_len > 0,
                AKV_ERR_SHAPE, "decode_step: unsupported extent (bsz %d, kv heads %d, group %d, head_dim %d [multiple "
                "of 64], max_seq_len %d)", B, H, G, D, max_seq_len);
    AKV_REQUIRE(rest_len >= 0 && rest_len < BLK && rest_start >= 0 && rest_start % BLK == 0 &&
                rest_start + rest_len + (append ? 1 : 0) <= max_seq_len, AKV_ERR_SHAPE,
                "decode_step: residual state (start %d, length %d) does not fit max_seq_len %d", rest_start, rest_len,
                max_seq_len);
    AKV_REQUIRE(!order_free || D == 128, AKV_ERR_SHAPE, "decode_step: the order-free P.V kernel needs head_dim 128");
    AKV_REQUIRE(scratch_bytes >= akv_decode_scratch_bytes_ex(B, H, G, D, max_seq_len, flags), AKV_ERR_SHAPE,
                "decode_step: scratch of %lld bytes is too small", scratch_bytes);
    AKV_REQUIRE(aligned16(scratch) && aligned16(q) && (!append || (aligned16(k_new) && aligned16(v_new))) &&
                (!out || aligned16(out)) && (!packed_out || aligned16(packed_out)) && aligned16(restk) &&
                aligned16(restv) && aligned16(k_exp_max) && aligned16(v_exp_max), AKV_ERR_ALIGN,
                "decode_step: pointers must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Scratch sc;
    carve(&sc, static_cast<uint8_t*>(scratch), B, H, G, D, max_seq_len, order_free);
    const int nmb = (max_seq_len + BLK - 1) / BLK;
    int rc;

    int rest = rest_len + (append ? 1 : 0), qn = rest_start;
    const bool flush = rest == BLK;
    // append and (when the residual buffer fills up) the flush of the block to the planes
    // (k_cache_file.py:102-118, v_cache_file.py:103-116): one launch when the block tile fits in default shared memory
    const bool fused_flush = flush && D <= 256 && aligned16(k_first_8) && aligned16(k_mid_4) && aligned16(k_last_4) &&
                             aligned16(v_first_8) && aligned16(v_mid_4) && aligned16(v_last_4);
    {
        const int blocks = fused_flush ? B * H * (2 + D / 64) : B * H;
        launch_chained(append_flush_kernel, dim3(blocks), dim3(128), fused_flush ? (size_t)BLK * 2 * D : 0, st,
            static_cast<uint32_t*>(restk), static_cast<uint32_t*>(restv), static_cast<uint16_t*>(k_exp_max),
            static_cast<uint16_t*>(v_exp_max), static_cast<const uint32_t*>(q), static_cast<const uint32_t*>(k_new),
            static_cast<const uint32_t*>(v_new), reinterpret_cast<uint16_t*>(sc.kq), sc.kqmax,
            static_cast<uint8_t*>(k_first_8), static_cast<uint8_t*>(k_mid_4), static_cast<uint8_t*>(k_last_4),
            static_cast<uint8_t*>(v_first_8), static_cast<uint8_t*>(v_mid_4), static_cast<uint8_t*>(v_last_4), B, H, G, D,
            rest_len, append ? 1 : 0, nmb, max_seq_len, qn);
        if ((rc = cuda_status(cudaGetLastError(), "decode_step append launch")) != AKV_OK) return rc;
    }
    if (flush) {
        if (!fused_flush) {
            rc = launch_k_save(static_cast<uint8_t*>(k_first_8), static_cast<uint8_t*>(k_mid_4),
                               static_cast<uint8_t*>(k_last_4), static_cast<const uint8_t*>(restk), B, H, 1, nmb, D, BLK,
                               qn, BLK, st);
            if (rc != AKV_OK) return rc;
            rc = launch_v_save(static_cast<uint8_t*>(v_first_8), static_cast<uint8_t*>(v_mid_4),
                               static_cast<uint8_t*>(v_last_4), static_cast<const uint8_t*>(restv), B, H, max_seq_len, D,
                               qn, BLK, BLK, st);
            if (rc != AKV_OK) return rc;
        }
        qn += BLK;
        rest = 0;
    }
    const int nb = qn / BLK;
    const int R = (nb + 1) * BLK;
    cudaEvent_t* ev = timing_slot();
    if (nb > 0) {
        if (ev) cudaEventRecord(ev[0], st);
        rc = launch_k_compute(static_cast<const uint8_t*>(k_first_8), static_cast<const uint8_t*>(k_mid_4),
                              static_cast<const uint8_t*>(k_last_4), sc.kq, sc.kqmax, static_cast<const uint8_t*>(q),
                              reinterpret_cast<uint8_t*>(sc.s), B, H, G, nb, nmb, D, BLK, 1.0f / sqrtf((float)D),
                              reference, st);
        if (ev) cudaEventRecord(ev[1], st);
        if (rc != AKV_OK) return rc;
    }
    // one CTA per row while there are enough rows to fill the GPU or the rows are short (three launches cost more
    // than they save below ~16k scores); else the split form
    const int sm_chunks = (R + SM_CHUNK - 1) / SM_CHUNK;
    bool probed = false;
    const int rows = B * H * G;
    const bool one_cta_512 = R > 256 * SM_REGS && R <= 512 * SM_REGS_512 && rows <= 2 * sm_count();
    const bool one_cta_256 = !one_cta_512 && !(sm_chunks >= 4 && rows < 2 * sm_count()) && R <= 256 * SM_REGS &&
                             rows <= 4 * sm_count();
    // The residual tokens' part of the output without a launch of its own: the softmax CTA of a row computes it beside
    // its probe (into o_main, as fp16), and the exact-order chain kernel adds it in its epilogue.
    const bool fuse_tail = !order_free && !packed_out && qn > 0 && rest > 0 && D <= 256 && (one_cta_512 || one_cta_256) &&
        v_compute_adds_residual(static_cast<const uint8_t*>(v_first_8), static_cast<const uint8_t*>(v_mid_4),
                                static_cast<const uint8_t*>(v_last_4), reinterpret_cast<const uint8_t*>(sc.s),
                                static_cast<const uint8_t*>(out), B, H, G, D, R, qn, reference);
    const __half* res_v = fuse_tail ? static_cast<const __half*>(restv) : nullptr;
    uint16_t* res_o = fuse_tail ? sc.o_main : nullptr;
    if (one_cta_512) {
        // few rows of up to 17408 scores: one CTA of 512 threads keeps the row in registers - one launch instead of the
        // four of the split form (statistics, probabilities, class reduction, probe)
        launch_chained(softmax_kernel<true, true, 512>, dim3(rows), dim3(512), 0, st, sc.s,
                       static_cast<const __half*>(q), static_cast<const __half*>(restk), sc.pval, sc.pidx, sc.stats,
                       static_cast<const uint8_t*>(v_first_8), sc.test_o, max_seq_len, H, G, D, R, qn, rest,
                       sqrtf((float)D), mk, mask_stride, res_v, res_o);
        probed = true;
    } else if (sm_chunks >= 4 && B * H * G < 2 * sm_count()) {
        dim3 grid(sm_chunks, B * H * G);
        count_launch();
        softmax_chunk_stats_kernel<<<grid, 256, 0, st>>>(sc.s, static_cast<const __half*>(q),
                                                        static_cast<const __half*>(restk), sc.cstat, H, G, D, R, qn, rest,
                                                        sqrtf((float)D), sm_chunks, mk, mask_stride);
        count_launch();
        softmax_chunk_write_kernel<<<grid, 256, 0, st>>>(sc.s, sc.cstat, sc.cand_val, sc.cand_idx, R, qn, qn + rest,
                                                        sm_chunks, sm_chunks, 1, 0, mk, mask_stride, H * G);
        count_launch();
        softmax_class_reduce_kernel<<<B * H * G, 32, 0, st>>>(sc.cstat, sc.cand_val, sc.cand_idx, sc.pval, sc.pidx,
                                                             sc.stats, sm_chunks, 1);
    } else {
        if (R <= 256 * SM_REGS && B * H * G <= 4 * sm_count()) {
            // few rows: one pass over the row, and the probe runs inside the softmax CTA of its row
            if (R <= 256 * 17)
                launch_chained(softmax_kernel<true, true, 256, 17>, dim3(B * H * G), dim3(256), 0, st, sc.s,
                               static_cast<const __half*>(q), static_cast<const __half*>(restk), sc.pval, sc.pidx,
                               sc.stats, static_cast<const uint8_t*>(v_first_8), sc.test_o, max_seq_len, H, G, D, R, qn,
                               rest, sqrtf((float)D), mk, mask_stride, res_v, res_o);
            else
                launch_chained(softmax_kernel<true, true, 256>, dim3(B * H * G), dim3(256), 0, st, sc.s,
                               static_cast<const __half*>(q), static_cast<const __half*>(restk), sc.pval, sc.pidx,
                               sc.stats, static_cast<const uint8_t*>(v_first_8), sc.test_o, max_seq_len, H, G, D, R, qn,
                               rest, sqrtf((float)D), mk, mask_stride, res_v, res_o);
            probed = true;
        } else {
            launch_chained(softmax_kernel<false, false, 256>, dim3(B * H * G), dim3(256), 0, st, sc.s,
                           static_cast<const __half*>(q), static_cast<const __half*>(restk), sc.pval, sc.pidx, sc.stats,
                           (const uint8_t*)nullptr, (uint16_t*)nullptr, max_seq_len, H, G, D, R, qn, rest,
                           sqrtf((float)D), mk, mask_stride, (const __half*)nullptr, (uint16_t*)nullptr);
        }
    }
    if ((rc = cuda_status(cudaGetLastError(), "decode_step softmax launch")) != AKV_OK) return rc;
    const bool need_tail = (rest > 0 && !fuse_tail) || qn == 0 || packed_out != nullptr || order_free;
    int v_chunks = 0;       // order-free P.V: chunk partials per row left for the tail kernel to add up
    if (qn > 0) {
        if (!probed) {
            rc = launch_v_probe(static_cast<const uint8_t*>(v_first_8), reinterpret_cast<const uint8_t*>(sc.pval),
                                reinterpret_cast<const uint8_t*>(sc.pidx), reinterpret_cast<uint8_t*>(sc.test_o), B, H,
                                G, max_seq_len, D, TOPK, st);
            if (rc != AKV_OK) return rc;
        }
        // the exact-order kernel derives the threshold bytes from the probe result in its prologue when it runs its
        // streaming form; otherwise a small kernel does
        const bool v_takes_probe = order_free
            ? v_split_takes_probe(G, reference, qn)
            : v_compute_takes_probe(static_cast<const uint8_t*>(v_first_8), static_cast<const uint8_t*>(v_mid_4),
                                    static_cast<const uint8_t*>(v_last_4), reinterpret_cast<const uint8_t*>(sc.s),
                                    need_tail ? (const uint8_t*)sc.o_main : (const uint8_t*)out, G, D, R, qn);
        if (!v_takes_probe) {
            launch_chained(amin_kernel, dim3((B * H * G + 3) / 4), dim3(128), 0, st, (const uint16_t*)sc.test_o,
                           static_cast<const uint8_t*>(v_exp_max), sc.amin, B * H * G, H, G, D);
            if ((rc = cuda_status(cudaGetLastError(), "decode_step threshold launch")) != AKV_OK) return rc;
        }
        if (ev) cudaEventRecord(ev[2], st);
        if (order_free)
            // the chunk partials stay in the workspace: the tail kernel adds them up (one launch less)
            rc = launch_v_split_probe(static_cast<const uint8_t*>(v_first_8), static_cast<const uint8_t*>(v_mid_4),
                                      static_cast<const uint8_t*>(v_last_4), reinterpret_cast<const uint8_t*>(sc.s),
                                      sc.amin, v_takes_probe ? (const uint8_t*)sc.test_o : nullptr,
                                      static_cast<const uint8_t*>(v_exp_max), nullptr, nullptr, sc.partial, &v_chunks, B,
                                      H, G, max_seq_len, D, R, qn, reference, st);
        else
            rc = launch_v_compute_res(static_cast<const uint8_t*>(v_first_8), static_cast<const uint8_t*>(v_mid_4),
                                      static_cast<const uint8_t*>(v_last_4), reinterpret_cast<const uint8_t*>(sc.s),
                                      sc.amin, v_takes_probe ? (const uint8_t*)sc.test_o : nullptr,
                                      static_cast<const uint8_t*>(v_exp_max),
                                      fuse_tail ? reinterpret_cast<const uint8_t*>(sc.o_main) : nullptr,
                                      reinterpret_cast<uint8_t*>(need_tail ? (void*)sc.o_main : out), B, H, G,
                                      max_seq_len, D, R, qn, reference, st);
        if (ev) cudaEventRecord(ev[3], st);
        if (rc != AKV_OK) return rc;
    } else if (order_free) {
        rc = cuda_status(cudaMemsetAsync(sc.o_main32, 0, (size_t)B * H * G * D * sizeof(float), st),
                         "decode_step clear");
        if (rc != AKV_OK) return rc;
    }
    if (need_tail) {
        launch_chained(tail_kernel, dim3(B * H * G), dim3(256), 0, st,
                       (const uint16_t*)((qn > 0 && !order_free) ? sc.o_main : nullptr),
                       (const float*)(order_free ? (v_chunks > 0 ? sc.partial : sc.o_main32) : nullptr), (const uint16_t*)sc.s,
                       static_cast<const __half*>(restv), static_cast<__half*>(out), (const float*)sc.stats,
                       static_cast<float*>(packed_out), H, G, D, R, qn, rest, v_chunks, xp);
        if ((rc = cuda_status(cudaGetLastError(), "decode_step tail launch")) != AKV_OK) return rc;
    }
    return AKV_OK;
}

// ------------------------------------------------------------------ decode step over a sequence shard, decision-exact
// One decode step of a cache whose sequence is split across devices, cut into four phases with an exchange between
// them, so that every shard takes the read decisions a single device holding the whole sequence would take:
//   phase 1  append (last shard) or take the new token into the exponent maxima only (AKV_STEP_NO_APPEND |
//            AKV_STEP_TRACK_MAXIMA), q.K^T over the local blocks, per 4096-score chunk the maximum and the sum of
//            exponentials                          -> exch_out: float [rows][local chunks][2]
// Layout of what is exchanged: a phase 1 / 2 output has a row stride of out_chunks chunks (0 = the local chunk count;
// a caller that pads every rank to the same count pre-fills the padding with empty chunks: statistics (-inf, 0),
// candidates 0).  A phase 2 / 3 input is n_ranks such buffers one after the other, as an all-gather leaves them
// (chunks_total = n_ranks x the common chunk count), or with n_ranks == 1 one buffer over all chunks.
//   phase 2  exch_in: float [rows][chunks_total][2], every shard's chunk statistics in sequence order.  Probabilities
//            with the whole row's maximum and sum, and per local chunk the candidates of the 32 residue classes with
//            positions in the whole sequence (token_base = position of local token 0, a multiple of 4096)
//                                                  -> exch_out: u32 value [rows][local chunks][32], then i32 position/32
//   phase 3  exch_in: the same two arrays over chunks_total.  Winners per class (largest probability, first
//            position); the high-byte rows of the winners this shard holds
//                                                  -> exch_out: bytes [rows][32][head_dim], zeros for rows held elsewhere
//   phase 4  exch_in: the shards' row buffers added up.  Probe, threshold bytes, order-free P.V over the local
//            tokens, residual tokens (last shard)  -> exch_out: float [rows][head_dim + 2], words 2.. = this shard's
//            part of the output (the parts add up to the output; words 0, 1 are unused)
// rows = bsz * n_kv_heads * group.  The chunk grid is the one a single device uses for its split softmax, and the sums
// are combined in the same order, so probabilities - and with them every read decision - come out bit-identical to a
// single device that takes the split path; the P.V partial sums differ only in how the fp32 additions are grouped.
// All phases take the state BEFORE the step (rest_len, rest_start); the caller updates it after phase 4 as for
// akv_decode_step_ex.  The workspace is the one of akv_decode_scratch_bytes_ex(..., AKV_STEP_ORDER_FREE).
int akv_shard_step(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                   void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q, const void* k_new,
                   const void* v_new, const void* exch_in, void* exch_out, void* scratch, long long scratch_bytes,
                   int bsz, int n_kv_heads, int group, int head_dim, int max_seq_len, int rest_len, int rest_start,
                   int token_base, int chunks_total, int n_ranks, int out_chunks, int flags, int phase, void* stream) {
    set_error("");
    const int B = bsz, H = n_kv_heads, G = group, D = head_dim;
    const bool reference = (flags & AKV_STEP_REFERENCE) != 0, append = (flags & AKV_STEP_NO_APPEND) == 0;
    const bool track = (flags & AKV_STEP_TRACK_MAXIMA) != 0;
    AKV_REQUIRE(k_first_8 && k_mid_4 && k_last_4 && v_first_8 && v_mid_4 && v_last_4 && k_exp_max && v_exp_max && restk &&
                restv && q && exch_out && scratch && (!(append || track) || (k_new && v_new)) && (phase == 1 || exch_in),
                AKV_ERR_NULL, "shard_step: null pointer");
    AKV_REQUIRE(B > 0 && H > 0 && G > 0 && G <= 8 && D == 128 && max_seq_len > 0 && phase >= 1 && phase <= 4 &&
                token_base >= 0 && token_base % SM_CHUNK == 0, AKV_ERR_SHAPE,
                "shard_step: unsupported extent (bsz %d, kv heads %d, group %d, head_dim %d [128], phase %d, token_base "
                "%d [multiple of %d])", B, H, G, D, phase, token_base, SM_CHUNK);
    AKV_REQUIRE(rest_len >= 0 && rest_len < BLK && rest_start >= 0 && rest_start % BLK == 0 &&
                rest_start + rest_len + (append ? 1 : 0) <= max_seq_len, AKV_ERR_SHAPE,
                "shard_step: residual state (start %d, length %d) does not fit max_seq_len %d", rest_start, rest_len,
                max_seq_len);
    AKV_REQUIRE(scratch_bytes >= akv_decode_scratch_bytes_ex(B, H, G, D, max_seq_len, AKV_STEP_ORDER_FREE), AKV_ERR_SHAPE,
                "shard_step: scratch of %lld bytes is too small", scratch_bytes);
    AKV_REQUIRE(aligned16(scratch) && aligned16(q) && aligned16(exch_out) && (!exch_in || aligned16(exch_in)) &&
                aligned16(restk) && aligned16(restv) && aligned16(k_exp_max) && aligned16(v_exp_max) &&
                (!k_new || aligned16(k_new)) && (!v_new || aligned16(v_new)) && aligned16(k_first_8) &&
                aligned16(k_mid_4) && aligned16(k_last_4) && aligned16(v_first_8) && aligned16(v_mid_4) &&
                aligned16(v_last_4), AKV_ERR_ALIGN, "shard_step: pointers must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Scratch sc;
    carve(&sc, static_cast<uint8_t*>(scratch), B, H, G, D, max_seq_len, true);
    const int nmb = (max_seq_len + BLK - 1) / BLK, rows = B * H * G;
    int rest = rest_len + (append ? 1 : 0), qn = rest_start;
    const bool flush = rest == BLK;
    if (flush) { qn += BLK; rest = 0; }
    const int nb = qn / BLK, R = (nb + 1) * BLK;
    const int chunks = (R + SM_CHUNK - 1) / SM_CHUNK;
    AKV_REQUIRE(phase == 1 || (chunks_total >= chunks && n_ranks >= 1 && chunks_total % n_ranks == 0), AKV_ERR_SHAPE,
                "shard_step: chunks_total %d (local chunks %d) in %d rank blocks", chunks_total, chunks, n_ranks);
    AKV_REQUIRE(out_chunks == 0 || out_chunks >= chunks, AKV_ERR_SHAPE, "shard_step: out_chunks %d < local chunks %d",
                out_chunks, chunks);
    const int oc = out_chunks ? out_chunks : chunks;      // row stride (in chunks) of the phase 1 / 2 outputs
    int rc;
    if (phase == 1) {
        const int blocks = flush ? B * H * (2 + D / 64) : B * H;
        launch_chained(append_flush_kernel, dim3(blocks), dim3(128), flush ? (size_t)BLK * 2 * D : 0, st,
            static_cast<uint32_t*>(restk), static_cast<uint32_t*>(restv), static_cast<uint16_t*>(k_exp_max),
            static_cast<uint16_t*>(v_exp_max), static_cast<const uint32_t*>(q), static_cast<const uint32_t*>(k_new),
            static_cast<const uint32_t*>(v_new), reinterpret_cast<uint16_t*>(sc.kq), sc.kqmax,
            static_cast<uint8_t*>(k_first_8), static_cast<uint8_t*>(k_mid_4), static_cast<uint8_t*>(k_last_4),
            static_cast<uint8_t*>(v_first_8), static_cast<uint8_t*>(v_mid_4), static_cast<uint8_t*>(v_last_4), B, H, G, D,
            rest_len, append ? 1 : (track ? 2 : 0), nmb, max_seq_len, rest_start);
        if ((rc = cuda_status(cudaGetLastError(), "shard_step append launch")) != AKV_OK) return rc;
        cudaEvent_t* slot = timing_slot();      // (timing: phase 4 of the same step records into the slot phase 1 took)
        g_shard_timing = slot;
        if (slot) cudaEventRecord(slot[0], st);
        if (nb > 0) {
            rc = launch_k_compute(static_cast<const uint8_t*>(k_first_8), static_cast<const uint8_t*>(k_mid_4),
                                  static_cast<const uint8_t*>(k_last_4), sc.kq, sc.kqmax, static_cast<const uint8_t*>(q),
                                  reinterpret_cast<uint8_t*>(sc.s), B, H, G, nb, nmb, D, BLK, 1.0f / sqrtf((float)D),
                                  reference, st);
            if (rc != AKV_OK) return rc;
        }
        if (slot) cudaEventRecord(slot[1], st);
        count_launch();
        softmax_chunk_stats_kernel<<<dim3(chunks, rows), 256, 0, st>>>(sc.s, static_cast<const __half*>(q),
            static_cast<const __half*>(restk), static_cast<float*>(exch_out), H, G, D, R, qn, rest, sqrtf((float)D), oc,
            (const __half*)nullptr, 0ll);
        return cuda_status(cudaGetLastError(), "shard_step statistics launch");
    }
    if (phase == 2) {
        uint32_t* val = static_cast<uint32_t*>(exch_out);
        count_launch();
        softmax_chunk_write_kernel<<<dim3(chunks, rows), 256, 0, st>>>(sc.s, static_cast<const float*>(exch_in), val,
            reinterpret_cast<int32_t*>(val + (size_t)rows * oc * TOPK), R, qn, qn + rest, oc, chunks_total, n_ranks,
            token_base, (const __half*)nullptr, 0ll, H * G);
        return cuda_status(cudaGetLastError(), "shard_step probabilities launch");
    }
    if (phase == 3) {
        const uint32_t* val = static_cast<const uint32_t*>(exch_in);
        count_launch(2);
        softmax_class_reduce_kernel<<<rows, 32, 0, st>>>(nullptr, val,
            reinterpret_cast<const int32_t*>(val + (size_t)rows * chunks_total * TOPK), sc.pval, sc.pidx, sc.stats,
            chunks_total, n_ranks);
        probe_rows_gather_kernel<<<rows, 128, 0, st>>>(static_cast<const uint8_t*>(v_first_8), sc.pidx,
            static_cast<uint8_t*>(exch_out), G, D, max_seq_len, qn, token_base);
        return cuda_status(cudaGetLastError(), "shard_step winners launch");
    }
    // phase 4
    count_launch();
    probe_from_rows_kernel<<<rows, 64, 0, st>>>(static_cast<const uint8_t*>(exch_in), sc.pval, sc.test_o, D);
    launch_chained(amin_kernel, dim3((rows + 3) / 4), dim3(128), 0, st, (const uint16_t*)sc.test_o,
                   static_cast<const uint8_t*>(v_exp_max), sc.amin, rows, H, G, D);
    if ((rc = cuda_status(cudaGetLastError(), "shard_step threshold launch")) != AKV_OK) return rc;
    cudaEvent_t* slot4 = tuning().timing ? g_shard_timing : nullptr;
    if (slot4) cudaEventRecord(slot4[2], st);
    if (qn > 0) {
        rc = launch_v_split(static_cast<const uint8_t*>(v_first_8), static_cast<const uint8_t*>(v_mid_4),
                            static_cast<const uint8_t*>(v_last_4), reinterpret_cast<const uint8_t*>(sc.s), sc.amin,
                            nullptr, sc.o_main32, sc.partial, B, H, G, max_seq_len, D, R, qn, reference, st);
        if (rc != AKV_OK) return rc;
    } else {
        rc = cuda_status(cudaMemsetAsync(sc.o_main32, 0, (size_t)rows * D * sizeof(float), st), "shard_step clear");
        if (rc != AKV_OK) return rc;
    }
    if (slot4) cudaEventRecord(slot4[3], st);
    g_shard_timing = nullptr;
    launch_chained(tail_kernel, dim3(rows), dim3(256), 0, st, (const uint16_t*)nullptr, (const float*)sc.o_main32,
                   (const uint16_t*)sc.s, static_cast<const __half*>(restv), static_cast<__half*>(nullptr),
                   (const float*)sc.stats, static_cast<float*>(exch_out), H, G, D, R, qn, rest, 0, XchgParams{});
    return cuda_status(cudaGetLastError(), "shard_step tail launch");
}

int akv_decode_step(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4, void* v_last_4,
                    void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q, const void* k_new,
                    const void* v_new, void* out, void* scratch, long long scratch_bytes, int bsz, int n_heads,
                    int head_dim, int max_seq_len, int rest_len, int rest_start, int reference, void* stream) {
    AKV_REQUIRE(out && k_new && v_new, AKV_ERR_NULL, "decode_step: null pointer");
    return akv_decode_step_ex(k_first_8, k_mid_4, k_last_4, v_first_8, v_mid_4, v_last_4, k_exp_max, v_exp_max, restk,
                              restv, q, k_new, v_new, out, nullptr, scratch, scratch_bytes, bsz, n_heads, 1, head_dim,
                              max_seq_len, rest_len, rest_start, reference ? AKV_STEP_REFERENCE : 0, stream);
}

int akv_rollback(void* k_mid_4, void* k_last_4, void* k_exp_max, void* v_exp_max, const void* k_exp_saved,
                 const void* v_exp_saved, int bsz, int n_kv_heads, int head_dim, int max_seq_len, int first_block,
                 int n_blocks, void* stream) {
    set_error("");
    AKV_REQUIRE(k_mid_4 && k_last_4 && k_exp_max && v_exp_max && k_exp_saved && v_exp_saved, AKV_ERR_NULL,
                "rollback: null pointer");
    const int nmb = (max_seq_len + BLK - 1) / BLK;
    AKV_REQUIRE(bsz > 0 && n_kv_heads > 0 && head_dim > 0 && head_dim % 16 == 0 && max_seq_len > 0 && first_block >= 0 &&
                n_blocks >= 0 && first_block + n_blocks <= nmb, AKV_ERR_SHAPE,
                "rollback: bad extent (bsz %d, heads %d, head_dim %d, blocks [%d, %d) of %d)", bsz, n_kv_heads, head_dim,
                first_block, first_block + n_blocks, nmb);
    AKV_REQUIRE(aligned16(k_mid_4) && aligned16(k_last_4) && aligned16(k_exp_max) && aligned16(v_exp_max) &&
                aligned16(k_exp_saved) && aligned16(v_exp_saved), AKV_ERR_ALIGN, "rollback: pointers must be 16-byte aligned");
    launch_chained(rollback_kernel, dim3(bsz * n_kv_heads), dim3(128), 0, static_cast<cudaStream_t>(stream),
        static_cast<uint4*>(k_mid_4), static_cast<uint4*>(k_last_4), static_cast<uint4*>(k_exp_max),
        static_cast<uint4*>(v_exp_max), static_cast<const uint4*>(k_exp_saved), static_cast<const uint4*>(v_exp_saved),
        head_dim, nmb, first_block, n_blocks);
    return cuda_status(cudaGetLastError(), "rollback launch");
}

int akv_lse_merge(const void* packed, void* out, int n_ranks, int rows, int head_dim, void* stream) {
    set_error("");
    AKV_REQUIRE(packed && out, AKV_ERR_NULL, "lse_merge: null pointer");
    AKV_REQUIRE(n_ranks > 0 && rows > 0 && head_dim > 0, AKV_ERR_SHAPE, "lse_merge: bad extent (%d ranks, %d rows, "
                "head_dim %d)", n_ranks, rows, head_dim);
    return launch_lse_merge(static_cast<const float*>(packed), static_cast<uint8_t*>(out), n_ranks, rows, head_dim,
                            static_cast<cudaStream_t>(stream));
}


// ------------------------------------------------------------------ decode step without any allocation
// Some callers may not allocate device memory at all: a serving process whose memory pool was carved up at start-up
// and whose allocator is locked afterwards, a plugin that runs inside somebody else's stream callback or real-time
// loop where cudaMalloc (which synchronises the device) is forbidden, or code that only holds raw pointers handed
// to it.  For them the workspace of the decode step lives in this library image instead: a fixed array in device
// global memory that every GPU loading the library reserves until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[AKV_NOALLOC_SCRATCH_BYTES];

namespace akv {
// Device address of g_noalloc_scratch per device ordinal.  In host code the array's name is only a handle for
// the runtime, not an address a kernel could use, so the address is looked up once per device (with that device
// current) and cached.
static void* g_noalloc_ptr[64] = {nullptr};

static int noalloc_workspace(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e, "decode_step_noalloc: cudaGetDevice");
    AKV_REQUIRE(dev >= 0 && dev < 64, AKV_ERR_SHAPE, "decode_step_noalloc: device ordinal %d is not supported", dev);
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return cuda_status(e, "decode_step_noalloc: cudaGetSymbolAddress");
        AKV_REQUIRE(p != nullptr, AKV_ERR_CUDA, "decode_step_noalloc: the workspace symbol has no device address");
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return AKV_OK;
}
}  // namespace akv

int akv_decode_step_noalloc(void* k_first_8, void* k_mid_4, void* k_last_4, void* v_first_8, void* v_mid_4,
                            void* v_last_4, void* k_exp_max, void* v_exp_max, void* restk, void* restv, const void* q,
                            const void* k_new, const void* v_new, void* out, int bsz, int n_heads, int head_dim,
                            int max_seq_len, int rest_len, int rest_start, int reference, void* stream) {
    set_error("");
    const long long need = akv_decode_scratch_bytes(bsz, n_heads, head_dim, max_seq_len);
    AKV_REQUIRE(need >= 0, AKV_ERR_SHAPE, "decode_step_noalloc: bad extent (bsz %d, heads %d, head_dim %d, "
                "max_seq_len %d)", bsz, n_heads, head_dim, max_seq_len);
    AKV_REQUIRE(need <= (long long)AKV_NOALLOC_SCRATCH_BYTES, AKV_ERR_SHAPE,
                "decode_step_noalloc: these extents need a %lld-byte workspace but the built-in one holds %lld bytes; "
                "use akv_decode_step with a caller-provided workspace", need, (long long)AKV_NOALLOC_SCRATCH_BYTES);
    void* ws = nullptr;
    int rc = noalloc_workspace(&ws);
    if (rc != AKV_OK) return rc;
    g_timing_off = true;      // the benchmark's per-kernel event brackets create events, which allocates: never here
    rc = akv_decode_step(k_first_8, k_mid_4, k_last_4, v_first_8, v_mid_4, v_last_4, k_exp_max, v_exp_max, restk, restv,
                         q, k_new, v_new, out, ws, (long long)AKV_NOALLOC_SCRATCH_BYTES, bsz, n_heads, head_dim,
                         max_seq_len, rest_len, rest_start, reference, stream);
    g_timing_off = false;
    return rc;
}

}  // extern "C"
