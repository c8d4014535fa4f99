// Exchange of the shards' packed results through peer memory (see akv_exchange.cuh): buffers, the stand-alone kernel
// and the device error flag of the exchange.  The decode step can run the same exchange at the end of its last
// kernel (akv_decode_step_exchange, akv_decode.cu).
#include "akv_exchange.cuh"

namespace akv {

static __device__ unsigned int g_xchg_wait_gave_up = 0;

__global__ void __launch_bounds__(128)
exchange_merge_kernel(const XchgParams p, const float* __restrict__ rec) {
    pdl_enter();
    __shared__ uint8_t* s_buf[XCHG_MAX_RANKS];
    __shared__ float s_rec[XCHG_ROW_FLOATS];
    exchange_merge_row(p, rec + (size_t)blockIdx.x * (p.D + 2), blockIdx.x, s_buf, s_rec);
}

int fill_exchange(XchgParams* p, void* const* bufs, int rank, int n_ranks, void* out, int rows, int head_dim,
                  unsigned int epoch, int timeout_ms) {
    AKV_REQUIRE(bufs && out, AKV_ERR_NULL, "exchange: null pointer");
    AKV_REQUIRE(n_ranks >= 1 && n_ranks <= XCHG_MAX_RANKS && rank >= 0 && rank < n_ranks, AKV_ERR_SHAPE,
                "exchange: rank %d of %d (at most %d ranks)", rank, n_ranks, XCHG_MAX_RANKS);
    AKV_REQUIRE(rows > 0 && head_dim > 0 && head_dim <= XCHG_MAX_D, AKV_ERR_SHAPE,
                "exchange: bad extent (%d rows, head_dim %d [at most %d])", rows, head_dim, XCHG_MAX_D);
    // every row's CTA has to be resident at once on every rank: a CTA that waits for a peer's row whose CTA waits for
    // a free SM behind CTAs that in turn wait for this rank could only end by the time limit
    AKV_REQUIRE(rows <= 2 * sm_count(), AKV_ERR_SHAPE, "exchange: %d rows are more than two per SM (%d SMs)", rows,
                sm_count());
    AKV_REQUIRE(epoch != 0, AKV_ERR_SHAPE, "exchange: epoch 0 is the buffers' initial state");
    AKV_REQUIRE(timeout_ms > 0 && timeout_ms <= 10000, AKV_ERR_SHAPE, "exchange: timeout of %d ms", timeout_ms);
    for (int g = 0; g < XCHG_MAX_RANKS; ++g) {
        p->bufs[g] = g < n_ranks ? static_cast<uint8_t*>(bufs[g]) : nullptr;
        AKV_REQUIRE(g >= n_ranks || (p->bufs[g] && aligned16(p->bufs[g])), AKV_ERR_NULL,
                    "exchange: buffer of rank %d is null or not 16-byte aligned", g);
    }
    static void* flag_of[64] = {nullptr};      // the flag's address on each device, looked up once
    int dev = 0;
    cudaGetDevice(&dev);
    void* err = dev >= 0 && dev < 64 ? flag_of[dev] : nullptr;
    if (!err) {
        cudaError_t e = cudaGetSymbolAddress(&err, g_xchg_wait_gave_up);
        if (e != cudaSuccess) return cuda_status(e, "exchange error flag");
        if (dev >= 0 && dev < 64) flag_of[dev] = err;
    }
    p->err = static_cast<unsigned int*>(err);
    p->out = static_cast<__half*>(out);
    p->rank = rank; p->R = n_ranks; p->rows = rows; p->D = head_dim;
    p->epoch = epoch;
    p->timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    return AKV_OK;
}

unsigned int exchange_error_flag(cudaError_t* e) {
    unsigned int v = 0;
    *e = cudaMemcpyFromSymbol(&v, g_xchg_wait_gave_up, sizeof(v));
    return v;
}
cudaError_t exchange_error_clear() {
    const unsigned int v = 0;
    return cudaMemcpyToSymbol(g_xchg_wait_gave_up, &v, sizeof(v));
}

}  // namespace akv

using namespace akv;

extern "C" long long akv_exchange_bytes(int n_ranks, int rows, int head_dim) {
    if (n_ranks < 1 || n_ranks > XCHG_MAX_RANKS || rows < 1 || head_dim < 1 || head_dim > XCHG_MAX_D) return -1;
    return (long long)exchange_buffer_bytes(n_ranks, rows, head_dim);
}

extern "C" int akv_peer_alloc(long long bytes, void** ptr, void* handle) {
    AKV_REQUIRE(ptr && handle, AKV_ERR_NULL, "peer_alloc: null pointer");
    AKV_REQUIRE(bytes > 0, AKV_ERR_SHAPE, "peer_alloc: %lld bytes", bytes);
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, (size_t)bytes);
    if (e != cudaSuccess) return cuda_status(e, "peer_alloc");
    e = cudaMemset(d, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d);
    if (e != cudaSuccess) {
        cudaFree(d);
        return cuda_status(e, "peer_alloc (IPC handle)");
    }
    static_assert(sizeof(h) == AKV_PEER_HANDLE_BYTES, "IPC handle size");
    memcpy(handle, &h, sizeof(h));
    *ptr = d;
    return AKV_OK;
}

extern "C" int akv_peer_open(const void* handle, void** ptr) {
    AKV_REQUIRE(ptr && handle, AKV_ERR_NULL, "peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* d = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_status(e, "peer_open");
    *ptr = d;
    return AKV_OK;
}

extern "C" int akv_peer_close(void* ptr) {
    if (!ptr) return AKV_OK;
    return cuda_status(cudaIpcCloseMemHandle(ptr), "peer_close");
}

extern "C" int akv_peer_free(void* ptr) {
    if (!ptr) return AKV_OK;
    return cuda_status(cudaFree(ptr), "peer_free");
}

extern "C" int akv_exchange_merge(void* const* bufs, int rank, int n_ranks, const void* record, void* out, int rows,
                                  int head_dim, unsigned int epoch, int timeout_ms, void* stream) {
    set_error("");
    AKV_REQUIRE(record, AKV_ERR_NULL, "exchange_merge: null pointer");
    XchgParams p;
    const int rc = fill_exchange(&p, bufs, rank, n_ranks, out, rows, head_dim, epoch, timeout_ms);
    if (rc != AKV_OK) return rc;
    cudaError_t e = launch_chained(exchange_merge_kernel, dim3(rows), dim3(128), 0, static_cast<cudaStream_t>(stream), p,
                                   static_cast<const float*>(record));
    return cuda_status(e, "exchange_merge launch");
}
