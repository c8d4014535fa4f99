/*
 * CPU oracle for the AlignedKV decode hot path.  TEST INFRASTRUCTURE ONLY: it is the checker that the parity
 * tests, the smoke check and the bench's cpu_baseline leg compare against; the product package never calls it.
 *
 * It restates, in plain scalar C, what the five reference operators compute on byte buffers laid out exactly
 * like the reference's tensors.  Every function cites the reference lines it follows (paths are relative to
 * the reference project root).  fp16 arithmetic is done as: exact product and sum in double, then ONE
 * round-to-nearest-even to binary16, which is what the GPU's fused fp16 multiply-add produces.
 *
 * Parity pin: the reference ships no tests or golden vectors.  This file is pinned by (1) known-answer vectors
 * derived from the bit-layout rules, (2) golden vectors produced by the reference's own CUDA kernels compiled
 * unmodified and run on a B200 (tests/golden/), and (3) live comparison against that compiled reference in the
 * GPU tests when it is present.
 */
#include <stdint.h>
#include <string.h>
#include <stddef.h>

typedef uint8_t u8;
typedef uint16_t u16;

/* ------------------------------------------------------------------ fp16 <-> double, single rounding */

double akvo_f16_to_f64(u16 h) {
    uint64_t sign = (uint64_t)(h & 0x8000) << 48;
    int exp = (h >> 10) & 0x1F;
    uint64_t man = h & 0x3FF;
    uint64_t bits;
    if (exp == 0x1F) {
        bits = sign | 0x7FF0000000000000ull | (man << 42);
    } else if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: value = man * 2^-24 */
            int e = -24;
            while (!(man & 0x400)) { man <<= 1; e--; }
            man &= 0x3FF;
            bits = sign | ((uint64_t)(e + 10 + 1023) << 52) | (man << 42);
        }
    } else {
        bits = sign | ((uint64_t)(exp - 15 + 1023) << 52) | (man << 42);
    }
    double d;
    memcpy(&d, &bits, 8);
    return d;
}

u16 akvo_f64_to_f16(double d) {
    uint64_t u;
    memcpy(&u, &d, 8);
    u16 sign = (u16)((u >> 48) & 0x8000);
    int bexp = (int)((u >> 52) & 0x7FF);
    uint64_t man = u & 0xFFFFFFFFFFFFFull;
    if (bexp == 0x7FF) return man ? 0x7FFF : (u16)(sign | 0x7C00); /* canonical NaN like the GPU */
    if (bexp == 0) return sign;                                    /* far below the fp16 range */
    int e = bexp - 1023;
    if (e > 15) return (u16)(sign | 0x7C00);
    man |= 1ull << 52;
    int shift = (e >= -14) ? 42 : 42 + (-14 - e);
    if (shift >= 64) return sign;
    uint64_t q = man >> shift;
    uint64_t rem = man & ((1ull << shift) - 1);
    uint64_t half = 1ull << (shift - 1);
    if (rem > half || (rem == half && (q & 1))) q++;
    uint32_t bits;
    if (e >= -14) bits = (uint32_t)((e + 15) << 10) + (uint32_t)(q - 1024); /* carry bumps the exponent */
    else bits = (uint32_t)q;                                               /* 1024 == smallest normal */
    if (bits >= 0x7C00) bits = 0x7C00;
    return (u16)(sign | bits);
}

/* round-to-nearest-even float -> half, the GPU's __float2half_rn */
u16 akvo_f32_to_f16(float f) { return akvo_f64_to_f16((double)f); }

/* fused multiply-add on binary16 bit patterns: round16(a*b + c) */
u16 akvo_hfma(u16 a, u16 b, u16 c) {
    double p = akvo_f16_to_f64(a) * akvo_f16_to_f64(b); /* exact: 22 significant bits */
    double r = p + akvo_f16_to_f64(c);                  /* exact wherever it can matter for the final rounding */
    return akvo_f64_to_f16(r);
}

u16 akvo_hmul(u16 a, u16 b) { return akvo_f64_to_f16(akvo_f16_to_f64(a) * akvo_f16_to_f64(b)); }

/* ------------------------------------------------------------------ plane reassembly (shared by K and V) */

/* even/odd member of a nibble pair: K_cache.cu:251-252, V_cache.cu:252-253 */
static inline u16 join_even(u8 first, u8 midb, u8 lastb) {
    return (u16)(((u16)first << 8) + (midb & 0xF0) + ((lastb & 0xF0) >> 4));
}
static inline u16 join_odd(u8 first, u8 midb, u8 lastb) {
    return (u16)(((u16)first << 8) + ((midb & 0x0F) << 4) + (lastb & 0x0F));
}

/* substitute bytes for planes that are not read: {0x00, 0x88} at K_cache.cu:201-205,249-250.
 * code 0: read mid and last; 1: read mid, last := 0x88; 2: mid := 0x88, last := 0x00 */
static inline void pick_planes(int code, u8 mid_in, u8 last_in, u8 *midb, u8 *lastb) {
    if (code == 0) { *midb = mid_in; *lastb = last_in; }
    else if (code == 1) { *midb = mid_in; *lastb = 0x88; }
    else { *midb = 0x88; *lastb = 0x00; }
}

/* ------------------------------------------------------------------ K planes: write */

/*
 * k_cache_save (K_cache.cu:97-164).  Planes: first_8 [B,H,nmb,D,d_block], mid_4/last_4 [B,H,nmb,D,d_block/2].
 * k_new: fp16 bytes [B,seqlen,H,D].  Branches: (start_pos==0 || seqlen%d_block==0) -> block writer over
 * n_blocks blocks starting at block start_pos/d_block (K_cache.cu:120-141, kernel :37-57); else seqlen==1 ->
 * single token at (start_pos/d_block, start_pos%d_block) (:142-161, kernel :83-93); anything else: no-op.
 * Nibbles are ADDED onto the existing byte (mod 256), the high byte is overwritten.
 */
void akvo_k_cache_save(u8 *first8, u8 *mid4, u8 *last4, const u8 *k_new, int bsz, int H, int n_blocks,
                       int n_max_blocks, int D, int d_block, int start_pos, int seqlen) {
    const int64_t hb = d_block >> 1;            /* nibble-plane row length */
    const int64_t st_blk = hb * D;              /* strides in nibble-plane bytes */
    const int64_t st_head = st_blk * n_max_blocks;
    const int64_t st_b = st_head * H;
    const int64_t in_tok = (int64_t)H * D;      /* k_new strides in elements */
    const int64_t in_b = in_tok * seqlen;
    if (start_pos == 0 || seqlen % d_block == 0) {
        if (n_blocks == 0) return;
        const int blk0 = start_pos / d_block;
        for (int b = 0; b < bsz; ++b)
            for (int h = 0; h < H; ++h)
                for (int z = 0; z < n_blocks; ++z) {
                    int t_lo = z * d_block;
                    int t_hi = t_lo + d_block < seqlen ? t_lo + d_block : seqlen;
                    for (int d = 0; d < D; ++d) {
                        int64_t row = b * st_b + h * st_head + (int64_t)(z + blk0) * st_blk + d * hb;
                        for (int t = t_lo; t < t_hi; ++t) {
                            int slot = t - t_lo;
                            const u8 *x = k_new + 2 * (b * in_b + t * in_tok + (int64_t)h * D + d);
                            int sh = (slot & 1) << 2;
                            first8[2 * row + slot] = x[1];
                            mid4[row + (slot >> 1)] += (u8)((x[0] & 0xF0) >> sh);
                            last4[row + (slot >> 1)] += (u8)((x[0] & 0x0F) << (4 - sh));
                        }
                    }
                }
    } else if (seqlen == 1) {
        const int blk = start_pos / d_block;
        const int slot = start_pos - blk * d_block;
        const int sh = (slot & 1) << 2;
        for (int b = 0; b < bsz; ++b)
            for (int h = 0; h < H; ++h)
                for (int d = 0; d < D; ++d) {
                    int64_t row = b * st_b + h * st_head + (int64_t)blk * st_blk + d * hb;
                    const u8 *x = k_new + 2 * (b * in_b + (int64_t)h * D + d);
                    first8[2 * row + slot] = x[1];
                    mid4[row + (slot >> 1)] += (u8)((x[0] & 0xF0) >> sh);
                    last4[row + (slot >> 1)] += (u8)((x[0] & 0x0F) << (4 - sh));
                }
    }
}

/* ------------------------------------------------------------------ K planes: aligned q.K^T */

/*
 * k_cache_compute (K_cache.cu:314-395, kernel :194-309).  For every quantized block and token:
 * acc = 0; for d in 0..D-1: acc = hfma(k~[t,d], q[d], acc); s = hmul(acc, half(sqrt_dim)).
 * Per (b,h,d): diff = (u8)(kqmax[b,h] - kq[b,h,d]); mid read iff diff<8, last read iff diff<4 (:211,249-250).
 * s_out: fp16 [B,H,(n_blocks+1)*d_block]; only [.., :n_blocks*d_block] is written (:330, :307-309).
 * codes_out (optional, [B,H,D]): 0 read both, 1 skip last, 2 skip both - the reference never materialises it.
 * The reference only computes heads below 4*floor(H/4) (:350); this oracle does the same.
 */
void akvo_k_cache_compute(const u8 *first8, const u8 *mid4, const u8 *last4, const u8 *kq, const u8 *kqmax,
                          const u16 *q, u16 *s_out, u8 *codes_out, int bsz, int H, int n_blocks,
                          int n_max_blocks, int D, int d_block, float sqrt_dim, int reference) {
    const int64_t hb = d_block >> 1;
    const int64_t st_blk = hb * D, st_head = st_blk * n_max_blocks, st_b = st_head * H;
    const int64_t s_head = (int64_t)(n_blocks + 1) * d_block, s_b = s_head * H;
    const u16 scale = akvo_f32_to_f16(sqrt_dim);
    const int H4 = (H >> 2) << 2;
    for (int b = 0; b < bsz; ++b)
        for (int h = 0; h < H4; ++h) {
            const u8 *kq_row = kq + ((int64_t)b * H + h) * D;
            const u8 top = kqmax[(int64_t)b * H + h];
            const u16 *q_row = q + ((int64_t)b * H + h) * D;
            for (int d = 0; d < D && codes_out; ++d) {
                u8 diff = (u8)(top - kq_row[d]);
                codes_out[((int64_t)b * H + h) * D + d] = reference ? 0 : (diff >= 8 ? 2 : (diff >= 4 ? 1 : 0));
            }
            for (int z = 0; z < n_blocks; ++z)
                for (int t = 0; t < d_block; ++t) {
                    u16 acc = 0;
                    for (int d = 0; d < D; ++d) {
                        u8 diff = (u8)(top - kq_row[d]);
                        int code = reference ? 0 : (diff >= 8 ? 2 : (diff >= 4 ? 1 : 0));
                        int64_t row = b * st_b + h * st_head + z * st_blk + d * hb;
                        u8 midb, lastb;
                        pick_planes(code, mid4[row + (t >> 1)], last4[row + (t >> 1)], &midb, &lastb);
                        u8 f = first8[2 * row + t];
                        u16 kbits = (t & 1) ? join_odd(f, midb, lastb) : join_even(f, midb, lastb);
                        acc = akvo_hfma(kbits, q_row[d], acc);
                    }
                    s_out[b * s_b + h * s_head + (int64_t)z * d_block + t] = akvo_hmul(acc, scale);
                }
        }
}

/* ------------------------------------------------------------------ V planes: write */

/*
 * v_cache_save (V_cache.cu:44-80, kernel :29-40).  Planes: first_8 [B,H,max_seq_len,D], mid_4/last_4
 * [B,H,max_seq_len,D/2]; v_new fp16 bytes [B,size1,H,D] where size1 is the tensor's own token extent (:65).
 * Plain stores; adjacent CHANNELS share a nibble byte (even channel in the high nibble).
 */
void akvo_v_cache_save(u8 *first8, u8 *mid4, u8 *last4, const u8 *v_new, int bsz, int H, int max_seq_len, int D,
                       int start_pos, int seq_len, int v_new_size1) {
    if (seq_len == 0) return;
    const int64_t hd = D >> 1;
    const int64_t st_head = hd * max_seq_len, st_b = st_head * H;
    const int64_t in_tok = (int64_t)H * D, in_b = in_tok * v_new_size1;
    for (int b = 0; b < bsz; ++b)
        for (int h = 0; h < H; ++h)
            for (int p = 0; p < seq_len; ++p) {
                int64_t row = b * st_b + h * st_head + (int64_t)(p + start_pos) * hd;
                const u8 *x = v_new + 2 * (b * in_b + p * in_tok + (int64_t)h * D);
                for (int c = 0; c < hd; ++c) {
                    u8 lo_e = x[4 * c], hi_e = x[4 * c + 1], lo_o = x[4 * c + 2], hi_o = x[4 * c + 3];
                    first8[2 * (row + c)] = hi_e;
                    first8[2 * (row + c) + 1] = hi_o;
                    mid4[row + c] = (u8)((lo_e & 0xF0) + ((lo_o & 0xF0) >> 4));
                    last4[row + c] = (u8)(((lo_e & 0x0F) << 4) + (lo_o & 0x0F));
                }
            }
}

/* ------------------------------------------------------------------ V planes: magnitude probe */

/*
 * v_cache_test_compute (V_cache.cu:125-168, kernel :104-122).  For j in 0..top_max_k-1:
 * row = idx[j]*top_max_k + j; acc = hfma(abs(half((first<<8)+0x80)), s_val[j], acc).  Output fp16 [B,H,D].
 * Row indices are used as given (the reference does not bounds-check; callers of this oracle must pass
 * in-range rows).
 */
void akvo_v_cache_test_compute(const u8 *first8, const u16 *s_val, const int32_t *s_idx, u16 *out, int bsz, int H,
                               int max_seq_len, int D, int top_max_k) {
    const int64_t st_head = (int64_t)D * max_seq_len, st_b = st_head * H;
    for (int b = 0; b < bsz; ++b)
        for (int h = 0; h < H; ++h)
            for (int d = 0; d < D; ++d) {
                u16 acc = 0;
                for (int j = 0; j < top_max_k; ++j) {
                    int64_t k = ((int64_t)b * H + h) * top_max_k + j;
                    int64_t rowi = (int64_t)s_idx[k] * top_max_k + j;
                    u8 f = first8[b * st_b + h * st_head + rowi * D + d];
                    u16 v = (u16)((0x0080 + ((u16)f << 8)) & 0x7FFF);
                    acc = akvo_hfma(v, s_val[k], acc);
                }
                out[((int64_t)b * H + h) * D + d] = acc;
            }
}

/* ------------------------------------------------------------------ V planes: aligned P.V */

/*
 * v_cache_compute (V_cache.cu:310-374, kernel :194-307).  Per (b,h): A = (int16)((int16)amin[b*H+h] << 10)
 * (wraps mod 2^16, :195-197); per token t < n: diff = (int16)(A - bits(s_t)); mid read iff diff < 0x0800,
 * last read iff diff < 0x0400 (:211,250-251); acc[d] = hfma(v~[t,d], s_t, acc[d]) for t in order (:203,304).
 * s is fp16 with head stride s_last_dim (:333); amin is read flat at b*H+h (:337).
 * codes_out (optional, [B,H,n]) as for K.
 */
void akvo_v_cache_compute(const u8 *first8, const u8 *mid4, const u8 *last4, const u16 *s, const u8 *amin,
                          u16 *o_out, u8 *codes_out, int bsz, int H, int max_seq_len, int D, int s_last_dim,
                          int n, int reference) {
    const int64_t hd = D >> 1;
    const int64_t st_head = hd * max_seq_len, st_b = st_head * H;
    for (int b = 0; b < bsz; ++b)
        for (int h = 0; h < H; ++h) {
            const u16 *s_row = s + ((int64_t)b * H + h) * s_last_dim;
            int16_t A = (int16_t)((u16)((u16)amin[(int64_t)b * H + h] << 10));
            u16 *o_row = o_out + ((int64_t)b * H + h) * D;
            for (int d = 0; d < D; ++d) o_row[d] = 0;
            for (int t = 0; t < n; ++t) {
                u16 sb = s_row[t];
                int16_t diff = (int16_t)((u16)A - sb);
                int code = reference ? 0 : (diff >= 0x0800 ? 2 : (diff >= 0x0400 ? 1 : 0));
                if (codes_out) codes_out[((int64_t)b * H + h) * n + t] = (u8)code;
                int64_t row = b * st_b + h * st_head + (int64_t)t * hd;
                for (int c = 0; c < hd; ++c) {
                    u8 midb, lastb;
                    pick_planes(code, mid4[row + c], last4[row + c], &midb, &lastb);
                    u16 ve = join_even(first8[2 * (row + c)], midb, lastb);
                    u16 vo = join_odd(first8[2 * (row + c) + 1], midb, lastb);
                    o_row[2 * c] = akvo_hfma(ve, sb, o_row[2 * c]);
                    o_row[2 * c + 1] = akvo_hfma(vo, sb, o_row[2 * c + 1]);
                }
            }
        }
}
