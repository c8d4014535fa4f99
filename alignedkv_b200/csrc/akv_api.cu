// extern "C" surface of libalignedkv_b200: argument validation, error text, dispatch to the launchers.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>

#include "akv_common.cuh"

namespace akv {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_status(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return AKV_OK;
    set_error("%s: %s", what, cudaGetErrorString(e));
    return AKV_ERR_CUDA;
}

struct DevInfo { int sms; int smem; };
static DevInfo dev_info() {
    static thread_local int cached_dev = -1;
    static thread_local DevInfo info = {148, 227 * 1024};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return info;
    if (dev != cached_dev) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) info.sms = v;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess && v > 0)
            info.smem = v;
        cached_dev = dev;
    }
    return info;
}
static Tuning g_tuning;
Tuning& tuning() { return g_tuning; }

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }
int sm_count() { return dev_info().sms; }
int max_dyn_smem() { return dev_info().smem; }

int launch_v_save(uint8_t*, uint8_t*, uint8_t*, const uint8_t*, int, int, int, int, int, int, int, cudaStream_t);
int launch_k_save(uint8_t*, uint8_t*, uint8_t*, const uint8_t*, int, int, int, int, int, int, int, int,
                  cudaStream_t);
int launch_k_compute(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*,
                     const uint8_t*, uint8_t*, int, int, int, int, int, int, int, float, int, cudaStream_t);
int launch_v_split(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*, float*,
                   float*, int, int, int, int, int, int, int, int, cudaStream_t);
long long v_split_scratch_bytes(int, int, int, int);
int launch_v_compute(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*,
                     int, int, int, int, int, int, int, int, cudaStream_t);
int launch_v_probe(const uint8_t*, const uint8_t*, const uint8_t*, uint8_t*, int, int, int, int, int, int,
                   cudaStream_t);

static bool fits_i64(long long a, long long b, long long c = 1, long long d = 1, long long e = 1) {
    // all factors are non-negative ints here; the plane kernels index with 64-bit offsets
    const long double lim = 9.0e18L;
    return (long double)a * b * c * d * e < lim;
}

}  // namespace akv

using namespace akv;
#define U8(p) reinterpret_cast<uint8_t*>(p)
#define CU8(p) reinterpret_cast<const uint8_t*>(p)

extern "C" {

int akv_abi_version(void) { return 1; }

const char* akv_last_error(void) { return g_err; }

long long akv_launch_count(void) { return akv::launches(); }

int akv_set_tuning(const char* key, int value) {
    g_err[0] = 0;
    AKV_REQUIRE(key, AKV_ERR_NULL, "set_tuning: null key");
    Tuning& t = tuning();
    if (!strcmp(key, "k_kch") && (value == 8 || value == 16)) t.k_kch = value;
    else if (!strcmp(key, "k_stages") && value >= 3 && value <= 6) t.k_stages = value;
    else if (!strcmp(key, "pdl") && (value == 0 || value == 1)) t.pdl = value;
    else if (!strcmp(key, "k_gqa_kch") && (value == 8 || value == 16)) t.k_gqa_kch = value;
    else if (!strcmp(key, "timing") && (value == 0 || value == 1)) t.timing = value;
    else if (!strcmp(key, "k_wpc") && value >= 0 && value <= 16) t.k_wpc = value;
    else if (!strcmp(key, "v_impl") && (value == 0 || value == 1)) t.v_impl = value;
    else if (!strcmp(key, "v_nf") && value >= 0 && value <= 16) t.v_nf = value;
    else if (!strcmp(key, "v_nside") && (value == 0 || value == 128 || value == 256 || value == 512))
        t.v_nside = value;
    else if (!strcmp(key, "v_cps") && value >= 0 && value <= 8) t.v_cps = value;
    else if (!strcmp(key, "v_gqa_form") && value >= 0 && value <= 2) t.v_gqa_form = value;
    else if (!strcmp(key, "v_npt") && value >= 0 && value <= 8) t.v_npt = value;
    else if (!strcmp(key, "v_split_impl") && (value == 0 || value == 1)) t.v_split_impl = value;
    else if (!strcmp(key, "v_ndw") && (value == 0 || value == 2 || value == 4)) t.v_ndw = value;
    else if (!strcmp(key, "v_split_nf") && (value == 0 || value == 4 || value == 8)) t.v_split_nf = value;
    else if (!strcmp(key, "v_split_cps") && value >= 0 && value <= 8) t.v_split_cps = value;
    else if (!strcmp(key, "v_upc") && value >= 0 && value <= 2) t.v_upc = value;
    else {
        set_error("set_tuning: unknown key or value out of range (%s = %d)", key, value);
        return AKV_ERR_SHAPE;
    }
    return AKV_OK;
}

int akv_k_cache_save(void* f8, void* m4, void* l4, const void* k_new, int bsz, int H, int n_blocks,
                     int n_max_blocks, int D, int d_block, int start_pos, int seqlen, void* stream) {
    g_err[0] = 0;
    AKV_REQUIRE(f8 && m4 && l4 && k_new, AKV_ERR_NULL, "k_cache_save: null pointer");
    AKV_REQUIRE(bsz > 0 && H > 0 && D > 0 && n_max_blocks > 0 && n_blocks >= 0 && seqlen >= 0 && start_pos >= 0,
                AKV_ERR_SHAPE, "k_cache_save: bad extent (bsz %d, heads %d, d_head %d, n_max_blocks %d, n_blocks %d, "
                "seqlen %d, start_pos %d)", bsz, H, D, n_max_blocks, n_blocks, seqlen, start_pos);
    AKV_REQUIRE(d_block >= 2 && d_block % 2 == 0, AKV_ERR_SHAPE, "k_cache_save: d_block %d must be even", d_block);
    AKV_REQUIRE(fits_i64(bsz, H, n_max_blocks, D, d_block) && fits_i64(bsz, H, D, (long long)seqlen + 1, 2),
                AKV_ERR_OVERFLOW, "k_cache_save: tensor extent overflows");
    if (start_pos == 0 || seqlen % d_block == 0) {
        AKV_REQUIRE(start_pos / d_block + n_blocks <= n_max_blocks, AKV_ERR_SHAPE,
                    "k_cache_save: blocks [%d, %d) exceed n_max_blocks %d", start_pos / d_block,
                    start_pos / d_block + n_blocks, n_max_blocks);
    } else if (seqlen == 1) {
        AKV_REQUIRE(start_pos / d_block < n_max_blocks, AKV_ERR_SHAPE,
                    "k_cache_save: position %d is outside %d blocks", start_pos, n_max_blocks);
    }
    return launch_k_save(U8(f8), U8(m4), U8(l4), CU8(k_new), bsz, H, n_blocks, n_max_blocks, D, d_block, start_pos,
                         seqlen, static_cast<cudaStream_t>(stream));
}

int akv_k_cache_compute(const void* f8, const void* m4, const void* l4, const void* kq, const void* kqmax,
                        const void* q, void* s_out, int bsz, int H, int n_blocks, int n_max_blocks, int D,
                        int d_block, int seqlen, float sqrt_dim, int reference, void* stream) {
    return akv_k_cache_compute_gqa(f8, m4, l4, kq, kqmax, q, s_out, bsz, H, 1, n_blocks, n_max_blocks, D, d_block,
                                   seqlen, sqrt_dim, reference, stream);
}

int akv_k_cache_compute_gqa(const void* f8, const void* m4, const void* l4, const void* kq, const void* kqmax,
                            const void* q, void* s_out, int bsz, int H, int group, int n_blocks, int n_max_blocks,
                            int D, int d_block, int seqlen, float sqrt_dim, int reference, void* stream) {
    (void)seqlen;  // carried for signature parity; the reference ignores it too
    g_err[0] = 0;
    AKV_REQUIRE(bsz > 0 && H > 0 && group > 0 && D > 0 && n_max_blocks > 0 && n_blocks >= 0, AKV_ERR_SHAPE,
                "k_cache_compute: bad extent (bsz %d, heads %d x %d, d_head %d, n_max_blocks %d, n_blocks %d)", bsz, H,
                group, D, n_max_blocks, n_blocks);
    AKV_REQUIRE(d_block >= 2 && d_block % 2 == 0, AKV_ERR_SHAPE, "k_cache_compute: d_block %d must be even",
                d_block);
    AKV_REQUIRE(n_blocks <= n_max_blocks, AKV_ERR_SHAPE, "k_cache_compute: n_blocks %d > n_max_blocks %d", n_blocks,
                n_max_blocks);
    if (n_blocks == 0) return AKV_OK;  // the reference returns its uninitialised buffer untouched
    AKV_REQUIRE(f8 && m4 && l4 && kq && kqmax && q && s_out, AKV_ERR_NULL, "k_cache_compute: null pointer");
    AKV_REQUIRE(fits_i64(bsz, H, n_max_blocks, D, d_block) &&
                fits_i64(bsz, (long long)H * group, (long long)n_blocks + 1, d_block, 2),
                AKV_ERR_OVERFLOW, "k_cache_compute: tensor extent overflows");
    AKV_REQUIRE((reinterpret_cast<uintptr_t>(q) & 1u) == 0 && (reinterpret_cast<uintptr_t>(s_out) & 1u) == 0,
                AKV_ERR_ALIGN, "k_cache_compute: q and s must be 2-byte aligned");
    return launch_k_compute(CU8(f8), CU8(m4), CU8(l4), CU8(kq), CU8(kqmax), CU8(q), U8(s_out), bsz, H, group, n_blocks,
                            n_max_blocks, D, d_block, sqrt_dim, reference != 0, static_cast<cudaStream_t>(stream));
}

int akv_v_cache_save(void* f8, void* m4, void* l4, const void* v_new, int bsz, int H, int max_seq_len, int D,
                     int start_pos, int seq_len, int v_new_tokens, void* stream) {
    g_err[0] = 0;
    if (seq_len == 0) return AKV_OK;  // V_cache.cu:54-55
    AKV_REQUIRE(f8 && m4 && l4 && v_new, AKV_ERR_NULL, "v_cache_save: null pointer");
    AKV_REQUIRE(bsz > 0 && H > 0 && D > 0 && D % 2 == 0 && max_seq_len > 0 && seq_len > 0 && start_pos >= 0 &&
                v_new_tokens >= seq_len, AKV_ERR_SHAPE,
                "v_cache_save: bad extent (bsz %d, heads %d, head_dim %d, max_seq_len %d, start_pos %d, seq_len %d, "
                "v_new tokens %d)", bsz, H, D, max_seq_len, start_pos, seq_len, v_new_tokens);
    AKV_REQUIRE((long long)start_pos + seq_len <= max_seq_len, AKV_ERR_SHAPE,
                "v_cache_save: tokens [%d, %d) exceed max_seq_len %d", start_pos, start_pos + seq_len, max_seq_len);
    AKV_REQUIRE(fits_i64(bsz, H, max_seq_len, D) && fits_i64(bsz, H, v_new_tokens, D, 2), AKV_ERR_OVERFLOW,
                "v_cache_save: tensor extent overflows");
    AKV_REQUIRE((reinterpret_cast<uintptr_t>(v_new) & 3u) == 0 && (reinterpret_cast<uintptr_t>(f8) & 1u) == 0,
                AKV_ERR_ALIGN, "v_cache_save: v_new must be 4-byte and first_8 2-byte aligned");
    return launch_v_save(U8(f8), U8(m4), U8(l4), CU8(v_new), bsz, H, max_seq_len, D, start_pos, seq_len,
                         v_new_tokens, static_cast<cudaStream_t>(stream));
}

int akv_v_cache_test_compute(const void* f8, const void* m4, const void* l4, const void* s_val, const void* s_idx,
                             void* test_o, int bsz, int H, int max_seq_len, int D, int top_max_k, void* stream) {
    (void)m4;
    (void)l4;  // the probe reads the high-byte plane only (V_cache.cu:111-112)
    g_err[0] = 0;
    AKV_REQUIRE(f8 && s_val && s_idx && test_o, AKV_ERR_NULL, "v_cache_test_compute: null pointer");
    AKV_REQUIRE(bsz > 0 && H > 0 && D > 0 && D % 2 == 0 && max_seq_len > 0 && top_max_k >= 0, AKV_ERR_SHAPE,
                "v_cache_test_compute: bad extent (bsz %d, heads %d, head_dim %d, max_seq_len %d, top_max_k %d)", bsz,
                H, D, max_seq_len, top_max_k);
    AKV_REQUIRE(fits_i64(bsz, H, max_seq_len, D), AKV_ERR_OVERFLOW, "v_cache_test_compute: tensor extent overflows");
    AKV_REQUIRE((reinterpret_cast<uintptr_t>(s_idx) & 3u) == 0 && (reinterpret_cast<uintptr_t>(test_o) & 3u) == 0 &&
                (reinterpret_cast<uintptr_t>(s_val) & 1u) == 0 && (reinterpret_cast<uintptr_t>(f8) & 1u) == 0,
                AKV_ERR_ALIGN, "v_cache_test_compute: misaligned pointer");
    return launch_v_probe(CU8(f8), CU8(s_val), CU8(s_idx), U8(test_o), bsz, H, 1, max_seq_len, D, top_max_k,
                          static_cast<cudaStream_t>(stream));
}

int akv_v_cache_compute(const void* f8, const void* m4, const void* l4, const void* s, const void* amin,
                        void* o_out, int bsz, int H, int max_seq_len, int D, int s_last_dim, int n, int reference,
                        void* stream) {
    return akv_v_cache_compute_gqa(f8, m4, l4, s, amin, o_out, nullptr, 0, bsz, H, 1, max_seq_len, D, s_last_dim, n,
                                   reference ? AKV_STEP_REFERENCE : 0, stream);
}

long long akv_v_cache_compute_scratch_bytes(int bsz, int n_kv_heads, int group, int n) {
    if (bsz <= 0 || n_kv_heads <= 0 || group <= 0 || n < 0) return -1;
    return v_split_scratch_bytes(bsz, n_kv_heads, group, n);
}

int akv_v_cache_compute_gqa(const void* f8, const void* m4, const void* l4, const void* s, const void* amin,
                            void* o_out, void* scratch, long long scratch_bytes, int bsz, int H, int group,
                            int max_seq_len, int D, int s_last_dim, int n, int flags, void* stream) {
    g_err[0] = 0;
    const bool reference = (flags & AKV_STEP_REFERENCE) != 0, order_free = (flags & AKV_STEP_ORDER_FREE) != 0;
    AKV_REQUIRE(f8 && m4 && l4 && amin && o_out && (s || n == 0), AKV_ERR_NULL, "v_cache_compute: null pointer");
    AKV_REQUIRE(bsz > 0 && H > 0 && group > 0 && D > 0 && D % 2 == 0 && max_seq_len > 0 && n >= 0 && s_last_dim >= 0,
                AKV_ERR_SHAPE, "v_cache_compute: bad extent (bsz %d, heads %d x %d, head_dim %d, max_seq_len %d, "
                "s_last_dim %d, tokens %d)", bsz, H, group, D, max_seq_len, s_last_dim, n);
    AKV_REQUIRE(n <= max_seq_len, AKV_ERR_SHAPE, "v_cache_compute: %d tokens exceed max_seq_len %d", n, max_seq_len);
    AKV_REQUIRE(n <= s_last_dim || bsz * H * group == 1, AKV_ERR_SHAPE,
                "v_cache_compute: %d tokens exceed the score row stride %d", n, s_last_dim);
    AKV_REQUIRE(fits_i64(bsz, H, max_seq_len, D) && fits_i64(bsz, (long long)H * group, s_last_dim, 2),
                AKV_ERR_OVERFLOW, "v_cache_compute: tensor extent overflows");
    AKV_REQUIRE((reinterpret_cast<uintptr_t>(s) & 1u) == 0 && (reinterpret_cast<uintptr_t>(o_out) & 3u) == 0 &&
                (reinterpret_cast<uintptr_t>(f8) & 1u) == 0, AKV_ERR_ALIGN, "v_cache_compute: misaligned pointer");
    if (order_free) {
        AKV_REQUIRE(scratch && scratch_bytes >= v_split_scratch_bytes(bsz, H, group, n), AKV_ERR_SHAPE,
                    "v_cache_compute (order-free): workspace of %lld bytes is too small", scratch_bytes);
        AKV_REQUIRE(n <= s_last_dim, AKV_ERR_SHAPE, "v_cache_compute (order-free): %d tokens exceed the row stride", n);
        return launch_v_split(CU8(f8), CU8(m4), CU8(l4), CU8(s), CU8(amin), U8(o_out), nullptr,
                              static_cast<float*>(scratch), bsz, H, group, max_seq_len, D, s_last_dim, n, reference,
                              static_cast<cudaStream_t>(stream));
    }
    return launch_v_compute(CU8(f8), CU8(m4), CU8(l4), CU8(s), CU8(amin), U8(o_out), bsz, H, group, max_seq_len, D,
                            s_last_dim, n, reference, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
