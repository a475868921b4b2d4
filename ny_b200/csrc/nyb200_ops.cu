// Stand-alone operators of the engine trait (binary64 product, fused transposed convolution of one group) and
// the cooperative deadline.  Host buffers in and out; the resident batch calls do not go through here.
#include <time.h>

#include "nyb200_internal.cuh"

namespace nyb {

static int64_t monotonic_ns() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (int64_t)ts.tv_sec * 1000000000LL + ts.tv_nsec;
}

bool deadline_passed(const nyb200_engine *e) { return e->deadline_ns >= 0 && monotonic_ns() >= e->deadline_ns; }

int deadline_abort(nyb200_engine *e, const char *where) {
    cudaStreamSynchronize(e->stream);  // launches already enqueued finish; nothing is interrupted
    e->batch.ran = false;
    e->batch.finished = false;
    return set_err(e, NYB200_ERR_DEADLINE, std::string("deadline passed during the ") + where);
}

namespace {

// C[m, n] = sum_k A[m, k] B[k, n] in binary64, one fused multiply-add chain per element in increasing k.
// 64 x 64 output tile per CTA, 16-deep K slices through shared memory, 4 x 4 elements per thread.
constexpr int TM = 64, TN = 64, TK = 16;
__global__ void __launch_bounds__(256)
k_dgemm(int M, int N, int K, const double *__restrict__ A, const double *__restrict__ B, double *__restrict__ C) {
    __shared__ double sA[TK][TM + 1], sB[TK][TN];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    double acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int t = threadIdx.x; t < TM * TK; t += 256) {
            int r = t / TK, kk = t % TK;
            sA[kk][r] = (m0 + r < M && k0 + kk < K) ? A[(long)(m0 + r) * K + k0 + kk] : 0.0;
        }
        for (int t = threadIdx.x; t < TK * TN; t += 256) {
            int kk = t / TN, c = t % TN;
            sB[kk][c] = (k0 + kk < K && n0 + c < N) ? B[(long)(k0 + kk) * N + n0 + c] : 0.0;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            double a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = sB[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) C[(long)m * N + n] = acc[i][j];
        }
}

}  // namespace

void launch_dgemm(nyb200_engine *e, int m, int n, int k, const double *a, const double *b, double *c) {
    dim3 grid((n + TN - 1) / TN, (m + TM - 1) / TM);
    k_dgemm<<<grid, 256, 0, e->stream>>>(m, n, k, a, b, c);
    e->launches++;
}

namespace {

// Transposed convolution of one group, product and scatter in one pass: every thread owns one input-side
// element (s, ic, iy, ix), walks the kernel taps whose output pixel exists and contracts over the output
// channels.  Lanes are consecutive ix, so for stride 1 a warp reads one contiguous run of pixels' channel
// vectors; the weights of a tap are shared by the warp.  Binary64 accumulation, one rounding to fp32.
__global__ void __launch_bounds__(256)
k_conv_transpose_group(nyb200_conv_transpose_params g, const float *__restrict__ A, const float *__restrict__ W,
                       float *__restrict__ out) {
    const long per_spec = (long)g.in_channels * g.in_h * g.in_w;
    const long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long)g.num_specs * per_spec) return;
    const int s = (int)(t / per_spec);
    long r = t - (long)s * per_spec;
    const int ic = (int)(r / ((long)g.in_h * g.in_w));
    r -= (long)ic * g.in_h * g.in_w;
    const int iy = (int)(r / g.in_w), ix = (int)(r - (long)iy * g.in_w);
    const int taps = g.in_channels * g.kernel_h * g.kernel_w;
    double acc = 0.0;
    for (int ky = 0; ky < g.kernel_h; ++ky) {
        const int ny = iy + g.pad_h - ky;
        if (ny < 0 || ny % g.stride_h) continue;
        const int oy = ny / g.stride_h;
        if (oy >= g.out_h) continue;
        for (int kx = 0; kx < g.kernel_w; ++kx) {
            const int nx = ix + g.pad_w - kx;
            if (nx < 0 || nx % g.stride_w) continue;
            const int ox = nx / g.stride_w;
            if (ox >= g.out_w) continue;
            const float *a = A + (((long)s * g.out_h + oy) * g.out_w + ox) * g.out_channels;
            const float *w = W + ((long)ic * g.kernel_h + ky) * g.kernel_w + kx;
            for (int oc = 0; oc < g.out_channels; ++oc) acc = fma((double)a[oc], (double)w[(long)oc * taps], acc);
        }
    }
    out[t] = (float)acc;
}

}  // namespace
}  // namespace nyb

using namespace nyb;

extern "C" {

int32_t nyb200_set_deadline_ns(nyb200_engine *e, int64_t ns_from_now) {
    if (!e) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    e->deadline_ns = ns_from_now < 0 ? -1 : monotonic_ns() + ns_from_now;
    return NYB200_OK;
}

int32_t nyb200_gemm_f64(nyb200_engine *e, int32_t m, int32_t k, int32_t n, const double *a, const double *b,
                        double *c_out) {
    if (!e || !a || !b || !c_out) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    if (m <= 0 || k <= 0 || n <= 0) return set_err(e, NYB200_ERR_SHAPE, "gemm_f64: non-positive dimension");
    NYB_CUDA(e, cudaSetDevice(e->device));
    NYB_DEADLINE(e, "binary64 product");
    NYB_WS(da, double *, e, "gemm_a", (size_t)m * k * 8);
    NYB_WS(db, double *, e, "gemm_b", (size_t)k * n * 8);
    NYB_WS(dc, double *, e, "gemm_c", (size_t)m * n * 8);
    NYB_CUDA(e, cudaMemcpyAsync(da, a, (size_t)m * k * 8, cudaMemcpyHostToDevice, e->stream));
    NYB_CUDA(e, cudaMemcpyAsync(db, b, (size_t)k * n * 8, cudaMemcpyHostToDevice, e->stream));
    dim3 grid((n + TN - 1) / TN, (m + TM - 1) / TM);
    k_dgemm<<<grid, 256, 0, e->stream>>>(m, n, k, da, db, dc);
    e->launches++;
    NYB_CUDA(e, cudaGetLastError());
    NYB_CUDA(e, cudaMemcpyAsync(c_out, dc, (size_t)m * n * 8, cudaMemcpyDeviceToHost, e->stream));
    NYB_CUDA(e, cudaStreamSynchronize(e->stream));
    return NYB200_OK;
}

int32_t nyb200_conv_transpose_2d(nyb200_engine *e, const float *a_reshaped, const float *weight_col,
                                 const nyb200_conv_transpose_params *params, float *out) {
    if (!e || !a_reshaped || !weight_col || !params || !out) return NYB200_ERR_INVALID;
    const nyb200_conv_transpose_params &g = *params;
    std::lock_guard<std::mutex> lk(e->mu);
    if (g.num_specs <= 0 || g.out_channels <= 0 || g.in_channels <= 0 || g.out_h <= 0 || g.out_w <= 0 || g.in_h <= 0 ||
        g.in_w <= 0 || g.kernel_h <= 0 || g.kernel_w <= 0 || g.stride_h <= 0 || g.stride_w <= 0 || g.pad_h < 0 || g.pad_w < 0)
        return set_err(e, NYB200_ERR_SHAPE, "conv_transpose_2d: non-positive dimension");
    // the forward convolution's geometry must be the one stated: out = (in + 2 pad - kernel) / stride + 1
    if ((g.in_h + 2 * g.pad_h - g.kernel_h) / g.stride_h + 1 != g.out_h || (g.in_w + 2 * g.pad_w - g.kernel_w) / g.stride_w + 1 != g.out_w ||
        g.in_h + 2 * g.pad_h < g.kernel_h || g.in_w + 2 * g.pad_w < g.kernel_w)
        return set_err(e, NYB200_ERR_SHAPE, "conv_transpose_2d: output size does not follow from input, kernel, stride and padding");
    NYB_CUDA(e, cudaSetDevice(e->device));
    NYB_DEADLINE(e, "transposed convolution");
    const size_t na = (size_t)g.num_specs * g.out_h * g.out_w * g.out_channels;
    const size_t nw = (size_t)g.out_channels * g.in_channels * g.kernel_h * g.kernel_w;
    const size_t no = (size_t)g.num_specs * g.in_channels * g.in_h * g.in_w;
    NYB_WS(da, float *, e, "gemm_a", na * 4);
    NYB_WS(dw, float *, e, "gemm_b", nw * 4);
    NYB_WS(dout, float *, e, "gemm_c", no * 4);
    NYB_CUDA(e, cudaMemcpyAsync(da, a_reshaped, na * 4, cudaMemcpyHostToDevice, e->stream));
    NYB_CUDA(e, cudaMemcpyAsync(dw, weight_col, nw * 4, cudaMemcpyHostToDevice, e->stream));
    k_conv_transpose_group<<<(unsigned)((no + 255) / 256), 256, 0, e->stream>>>(g, da, dw, dout);
    e->launches++;
    NYB_CUDA(e, cudaGetLastError());
    NYB_CUDA(e, cudaMemcpyAsync(out, dout, no * 4, cudaMemcpyDeviceToHost, e->stream));
    NYB_CUDA(e, cudaStreamSynchronize(e->stream));
    return NYB200_OK;
}

}  // extern "C"
