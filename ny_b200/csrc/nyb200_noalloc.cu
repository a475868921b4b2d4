// nyb200_ibp_forward_noalloc: the single-box interval forward pass with its scratch in a fixed,
// library-owned device array, for callers that must not allocate device memory.
//
// Who needs it.  The other entry points keep a grow-only workspace and may call cudaMalloc the first
// time a shape is seen.  Some hosts cannot tolerate that: a verifier embedded in a service that hands
// every free byte of the GPU to its own arena at start-up (a later cudaMalloc simply fails there), or
// a BaB driver whose latency budget excludes the device-wide synchronisation that cudaMalloc/cudaFree
// imply.  For them this one call needs nothing beyond what the library image already carries.
//
// What it costs.  The scratch below is part of the loaded module: every GPU on which this library is
// used holds NYB200_NOALLOC_MAX_WIDTH * 4 floats + 256 bytes (about 128 KB) from first use until the
// process exits, whether or not this entry point is ever called.
//
// Rules for callers (also stated at the declaration in include/nyb200.h):
//   * Linear layers without residual connections only: a network with a Conv2d layer or a skip is refused
//     (NYB200_ERR_UNSUPPORTED) before any launch;
//   * layer widths (including the input width) above NYB200_NOALLOC_MAX_WIDTH are refused;
//   * all calls on one GPU share the same scratch: two calls that overlap on the device (different
//     streams or engines) race on it and both results are undefined; calls on one stream are ordered
//     and safe.  Nothing in the scratch needs a particular initial value except the status word, which
//     every call clears first; the interval buffers are fully rewritten for the widths in use, so the
//     previous call's leftovers are never read;
//   * the first call on a GPU looks up the scratch's device address (cudaGetSymbolAddress).  Make that
//     first call outside any stream capture.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "nyb200_internal.cuh"

#define NYB200_NOALLOC_MAX_WIDTH 8192

namespace {

// [0, 64): status words; then two pairs of interval vectors (lower ends, upper ends) of MAX_WIDTH floats
// each: a layer reads one pair (or the caller's box) and writes the other.
static __device__ __align__(256) float g_noalloc_scratch[64 + 4 * NYB200_NOALLOC_MAX_WIDTH];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float *g_scratch_addr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle; the address a kernel can use is obtained once per
// device, with that device current.
cudaError_t scratch_for_current_device(int device, float **out) {
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_scratch_addr[device]) {
        void *p = nullptr;
        cudaError_t st = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (st != cudaSuccess) return st;
        g_scratch_addr[device] = (float *)p;
    }
    *out = g_scratch_addr[device];
    return cudaSuccess;
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Interval image of one Linear layer for one box (same arithmetic as the engine's single-box kernel:
// exact fp32 products accumulated in binary64, one warp per output neuron, outward directed cast), followed
// by the ReLU on the interval: the pre-activation ends go to the caller's output, the post-activation
// ends to the scratch vectors the next layer reads.
__global__ void __launch_bounds__(256)
k_noalloc_layer(int n_in, int n_out, int relu, const float *__restrict__ W, const float *__restrict__ bias,
                const float *__restrict__ zl, const float *__restrict__ zu, float *__restrict__ pre_lo,
                float *__restrict__ pre_hi, float *__restrict__ next_l, float *__restrict__ next_u, int *status) {
    int o = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (o >= n_out) return;
    const float *w = W + (long)o * n_in;
    double lo = 0.0, hi = 0.0, qq = 0.0;
    for (int i = lane; i < n_in; i += 32) {
        double wv = w[i], a = zl[i], b = zu[i];
        bool pos = wv > 0.0;
        lo = fma(wv, pos ? a : b, lo);
        hi = fma(wv, pos ? b : a, hi);
        qq = fma(fabs(wv), fmax(fabs(a), fabs(b)), qq);
    }
    lo = warp_sum_d(lo); hi = warp_sum_d(hi); qq = warp_sum_d(qq);
    if (lane == 0) {
        const double gam = (double)(n_in + 2) * 1.1102230246251565e-16 * 1.000001;
        double bv = bias ? (double)bias[o] : 0.0;
        double slack = gam * (qq + fabs(bv));
        float lf = __double2float_rd(lo + bv - slack), hf = __double2float_ru(hi + bv + slack);
        if (isnan(lf) || isnan(hf)) { lf = -INFINITY; hf = INFINITY; }
        if (!isfinite(lf) || !isfinite(hf)) atomicExch(status, 1);
        pre_lo[o] = lf; pre_hi[o] = hf;
        if (relu) { next_l[o] = fmaxf(lf, 0.f); next_u[o] = fmaxf(hf, 0.f); }
    }
}

}  // namespace

extern "C" int32_t nyb200_ibp_forward_noalloc(nyb200_engine *e, int32_t net_id, const float *dev_in_lo,
                                              const float *dev_in_hi, float *dev_pre_lo, float *dev_pre_hi) {
    if (!e || !dev_in_lo || !dev_in_hi || !dev_pre_lo || !dev_pre_hi) return NYB200_ERR_INVALID;
    std::lock_guard<std::mutex> g(e->mu);
    auto it = e->nets.find(net_id);
    if (it == e->nets.end()) return nyb::set_err(e, NYB200_ERR_INVALID, "unknown net id");
    const nyb::Net &net = it->second;
    const nyb::NetView &nv = net.v;
    // The layer kernel below is a dense mat-vec over W[n_out x n_in]: a Conv2d layer stores only its
    // [out_channels x in_channels*kh*kw] filter bank and a residual layer needs the skipped activation,
    // so both are refused here, before anything is launched.
    for (int k = 0; k < nv.L; ++k) {
        if (net.is_conv(k))
            return nyb::set_err(e, NYB200_ERR_UNSUPPORTED,
                                "nyb200_ibp_forward_noalloc: layer " + std::to_string(k) +
                                    " is a Conv2d layer; only Linear layers without skips are supported, use nyb200_ibp_forward");
        if (net.skip_of(k) >= 0)
            return nyb::set_err(e, NYB200_ERR_UNSUPPORTED,
                                "nyb200_ibp_forward_noalloc: layer " + std::to_string(k) +
                                    " takes a residual connection; only Linear layers without skips are supported, use nyb200_ibp_forward");
    }
    for (int k = 0; k <= nv.L; ++k)
        if (nv.dims[k] > NYB200_NOALLOC_MAX_WIDTH)
            return nyb::set_err(e, NYB200_ERR_UNSUPPORTED,
                                "nyb200_ibp_forward_noalloc: layer width " + std::to_string(nv.dims[k]) +
                                    " exceeds the fixed scratch (" + std::to_string(NYB200_NOALLOC_MAX_WIDTH) +
                                    " per layer); use nyb200_ibp_forward");
    cudaError_t st = cudaSetDevice(e->device);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaSetDevice");
    float *scratch = nullptr;
    st = scratch_for_current_device(e->device, &scratch);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaGetSymbolAddress(scratch)");
    int *status = (int *)scratch;
    float *pair[2][2] = {{scratch + 64, scratch + 64 + NYB200_NOALLOC_MAX_WIDTH},
                         {scratch + 64 + 2 * NYB200_NOALLOC_MAX_WIDTH, scratch + 64 + 3 * NYB200_NOALLOC_MAX_WIDTH}};
    st = cudaMemsetAsync(status, 0, 256, e->stream);  // the only part of the scratch that must start at zero
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "cudaMemsetAsync(status)");
    const float *cur_l = dev_in_lo, *cur_u = dev_in_hi;
    for (int k = 0; k < nv.L; ++k) {
        int n_in = nv.dims[k], n_out = nv.dims[k + 1];
        int relu = (k < nv.L - 1) ? 1 : 0;
        float *nl = pair[k & 1][0], *nu = pair[k & 1][1];  // layer k reads pair (k-1)&1 (or the input), writes pair k&1
        k_noalloc_layer<<<(n_out * 32 + 255) / 256, 256, 0, e->stream>>>(n_in, n_out, relu, nv.W[k], nv.b[k], cur_l, cur_u,
                                                                        dev_pre_lo + nv.pre_off[k],
                                                                        dev_pre_hi + nv.pre_off[k], nl, nu, status);
        e->launches++;
        cur_l = nl; cur_u = nu;
    }
    st = cudaGetLastError();
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "k_noalloc_layer");
    int host_status = 0;
    st = cudaMemcpyAsync(&host_status, status, sizeof(int), cudaMemcpyDeviceToHost, e->stream);
    if (st == cudaSuccess) st = cudaStreamSynchronize(e->stream);
    if (st != cudaSuccess) return nyb::check_cuda(e, st, "nyb200_ibp_forward_noalloc: stream");
    if (host_status) return nyb::set_err(e, NYB200_ERR_NUMERICAL, "non-finite interval bound in the forward pass");
    return NYB200_OK;
}
