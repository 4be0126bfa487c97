// qagg_capi.cu -- C entry points for layout helpers and the single-matrix quantizer (include/qagg.h).
#include "../../include/qagg.h"
#include "qagg_internal.h"

#include <mutex>
#include <string>

namespace qagg {

static thread_local std::string g_lastError;

int fail(int code, const std::string& msg)
{
    g_lastError = msg;
    return code;
}

int check_cuda(cudaError_t e, const char* what)
{
    if (e == cudaSuccess)
        return QAGG_OK;
    return fail(QAGG_ECUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

bool bits_ok(int bits)
{
    return bits == 1 || bits == 2 || bits == 4 || bits == 8 || bits == 16 || bits == 32;
}

int mode_of(int bits, int zeroThr)
{
    if (bits == 1)
        return zeroThr ? MODE_ONEBIT_ZERO : MODE_ONEBIT_MEAN;
    return MODE_MULTIBIT;
}

void fill_layout(QTensor* t, long long M, long long N, int bits)
{
    t->M = M;
    t->N = N;
    t->bits = bits;
    t->Q = (int) ((M * bits + 31) / 32);
    t->colBytes = 8 + 4 * t->Q;
    t->K = 1;
    t->per = N;
    t->rem = 0;
}

// per-device launch configuration, looked up once
int launch_cfg_for_current_device(LaunchCfg* cfg)
{
    static std::mutex mu;
    static LaunchCfg cache[64];
    static bool have[64] = {};
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc)
        return rc;
    if (dev < 0 || dev >= 64)
        return fail(QAGG_EINVAL, "device index out of range");
    std::lock_guard<std::mutex> lk(mu);
    if (!have[dev])
    {
        rc = check_cuda(get_launch_cfg(dev, &cache[dev]), "cudaGetDeviceProperties");
        if (rc)
            return rc;
        have[dev] = true;
    }
    *cfg = cache[dev];
    return QAGG_OK;
}

int check_dims(long long M, long long N, int bits)
{
    if (!bits_ok(bits))
        return fail(QAGG_EINVAL, "bits must be a power of two in 1..32");
    if (M < 0 || N < 0)
        return fail(QAGG_EINVAL, "negative matrix dimension");
    if (M > 0x7fffffffLL / 2 || N > 0x7fffffffLL)
        return fail(QAGG_EINVAL, "matrix dimension too large (rows < 2^30, columns < 2^31)");
    return QAGG_OK;
}

} // namespace qagg

using namespace qagg;

extern "C" {

const char* qagg_last_error(void)
{
    return g_lastError.c_str();
}

int qagg_abi_version(void)
{
    return 2;
}

int64_t qagg_packed_col_bytes(int64_t M, int bits)
{
    if (!bits_ok(bits) || M < 0)
        return fail(QAGG_EINVAL, "qagg_packed_col_bytes: bad arguments");
    return 8 + 4 * ((M * bits + 31) / 32);
}

int64_t qagg_packed_bytes(int64_t M, int64_t N, int bits)
{
    if (!bits_ok(bits) || M < 0 || N < 0)
        return fail(QAGG_EINVAL, "qagg_packed_bytes: bad arguments");
    return N * (8 + 4 * ((M * bits + 31) / 32));
}

int qagg_stripe(int64_t num_cols, int rank, int num_ranks, int64_t* start_col, int64_t* n)
{
    if (num_cols < 0 || num_ranks < 1 || rank < 0 || rank >= num_ranks || !start_col || !n)
        return fail(QAGG_EINVAL, "qagg_stripe: bad arguments");
    const int64_t per = num_cols / num_ranks;
    const int64_t rem = num_cols % num_ranks;
    *start_col = per * rank + (rem < rank ? rem : rank);
    *n = per + ((rank < rem) ? 1 : 0);
    return QAGG_OK;
}

int qagg_quantize(void* stream, const float* grad, const float* res_in, float* res_out, void* packed,
                  int64_t M, int64_t N, int bits, int zero_threshold)
{
    int rc = check_dims(M, N, bits);
    if (rc)
        return rc;
    if (M == 0 || N == 0)
        return QAGG_OK;
    if (!grad || !res_in || !res_out || !packed)
        return fail(QAGG_EINVAL, "qagg_quantize: null pointer");
    if ((reinterpret_cast<uintptr_t>(packed) & 3) || (reinterpret_cast<uintptr_t>(grad) & 3))
        return fail(QAGG_EINVAL, "qagg_quantize: buffers must be 4-byte aligned");
    LaunchCfg cfg;
    rc = launch_cfg_for_current_device(&cfg);
    if (rc)
        return rc;
    QTensor t = {};
    fill_layout(&t, M, N, bits);
    t.grad = grad;
    t.res_in = res_in;
    t.res_out = res_out;
    t.pk[0] = static_cast<unsigned char*>(packed);
    const int c = cols_per_item(M, N, cfg.smemFloats, nullptr);
    const int nItems = (int) ((N + c - 1) / c);
    return check_cuda(launch_colquant((cudaStream_t) stream, false, mode_of(bits, zero_threshold), &t, nullptr, nullptr, nItems, c, cfg),
                      "quantize kernel launch");
}

int qagg_unquantize(void* stream, const void* packed, float* out, int64_t M, int64_t N, int bits, int add)
{
    int rc = check_dims(M, N, bits);
    if (rc)
        return rc;
    if (M == 0 || N == 0)
        return QAGG_OK;
    if (!packed || !out)
        return fail(QAGG_EINVAL, "qagg_unquantize: null pointer");
    LaunchCfg cfg;
    rc = launch_cfg_for_current_device(&cfg);
    if (rc)
        return rc;
    QTensor t = {};
    fill_layout(&t, M, N, bits);
    t.out = out;
    t.pk[0] = static_cast<unsigned char*>(const_cast<void*>(packed));
    return check_cuda(launch_unquantize((cudaStream_t) stream, add != 0 ? UNQ_ADD : UNQ_STORE, bits, &t, nullptr, 1, unq_units(M, N, bits), unq_smem_words(M, bits), cfg), "unquantize kernel launch");
}

int qagg_reduce_requantize(void* stream, const void* const* stripes, int K, const float* self_raw,
                           const float* sres_in, float* sres_out, void* packed_out,
                           int64_t M, int64_t n, int bits, int zero_threshold)
{
    int rc = check_dims(M, n, bits);
    if (rc)
        return rc;
    if (K < 1 || K > QAGG_MAXK)
        return fail(QAGG_EINVAL, "qagg_reduce_requantize: K out of range");
    if (M == 0 || n == 0)
        return QAGG_OK;
    if (!stripes || !sres_in || !sres_out || !packed_out)
        return fail(QAGG_EINVAL, "qagg_reduce_requantize: null pointer");
    LaunchCfg cfg;
    rc = launch_cfg_for_current_device(&cfg);
    if (rc)
        return rc;
    QTensor t = {};
    fill_layout(&t, M, n, bits);
    t.grad = self_raw;
    t.selfRaw = self_raw ? 1 : 0;
    t.res_in = sres_in;
    t.res_out = sres_out;
    t.pk[0] = static_cast<unsigned char*>(packed_out);
    t.nsrc = K;
    for (int s = 0; s < K; ++s)
    {
        t.src[s] = static_cast<const unsigned char*>(stripes[s]);
        if (!t.src[s] && !(s == 0 && self_raw))
            return fail(QAGG_EINVAL, "qagg_reduce_requantize: null stripe pointer");
    }
    const int c = cols_per_item(M, n, cfg.smemFloats, nullptr);
    const int nItems = (int) ((n + c - 1) / c);
    return check_cuda(launch_colquant((cudaStream_t) stream, true, mode_of(bits, zero_threshold), &t, nullptr, nullptr, nItems, c, cfg),
                      "reduce-requantize kernel launch");
}

int qagg_quantize_to_host(void* stream, const float* grad, const float* res_in, float* res_out, void* dev_scratch,
                          void* host_packed, int64_t M, int64_t N, int bits, int zero_threshold)
{
    int rc = qagg_quantize(stream, grad, res_in, res_out, dev_scratch, M, N, bits, zero_threshold);
    if (rc)
        return rc;
    if (M == 0 || N == 0)
        return QAGG_OK;
    if (!host_packed)
        return fail(QAGG_EINVAL, "qagg_quantize_to_host: null host buffer");
    rc = check_cuda(cudaMemcpyAsync(host_packed, dev_scratch, (size_t) qagg_packed_bytes(M, N, bits), cudaMemcpyDeviceToHost, (cudaStream_t) stream),
                    "copy of packed matrix to host");
    if (rc)
        return rc;
    return check_cuda(cudaStreamSynchronize((cudaStream_t) stream), "cudaStreamSynchronize");
}

int qagg_unquantize_from_host(void* stream, const void* host_packed, void* dev_scratch, float* out,
                              int64_t M, int64_t N, int bits, int add)
{
    int rc = check_dims(M, N, bits);
    if (rc)
        return rc;
    if (M == 0 || N == 0)
        return QAGG_OK;
    if (!host_packed || !dev_scratch)
        return fail(QAGG_EINVAL, "qagg_unquantize_from_host: null buffer");
    rc = check_cuda(cudaMemcpyAsync(dev_scratch, host_packed, (size_t) qagg_packed_bytes(M, N, bits), cudaMemcpyHostToDevice, (cudaStream_t) stream),
                    "copy of packed matrix to device");
    if (rc)
        return rc;
    rc = qagg_unquantize(stream, dev_scratch, out, M, N, bits, add);
    if (rc)
        return rc;
    return check_cuda(cudaStreamSynchronize((cudaStream_t) stream), "cudaStreamSynchronize");
}

} // extern "C"
