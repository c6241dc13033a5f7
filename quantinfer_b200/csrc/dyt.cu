// Dynamic tanh in place of a norm, with the residual update fused in:
//
//     dyt(v) = tanh(alpha * v) * w + b          elementwise; alpha one number, w and b per coordinate
//
// It needs no statistic of its row, so everything around a sublayer that is elementwise rides in one
// launch: the sublayer's output y (with the bias of its last projection, if that was left unapplied)
// goes through a post-norm and a multiplier into the 32-bit residual stream, and the stream's new value
// goes through the pre-norm of the next sublayer:
//
//     t = y + y_bias ;  t = mult * dyt_post(t)  (when a post-norm is given) ;  x = resid + t ;  resid = x
//     out = dyt_pre(x)                           (when a pre-norm is given)
//
// y may also be the 32-bit partial sums [splits, n, h] of a projection whose product was cut along K; they are
// added here, in split order. `rows` gathers source rows (the head reads only the wanted places; the stream is then not written).
// All arithmetic is 32-bit; y and out may be bfloat16. alpha is read from device memory (a tensor of
// shape []), so nothing crosses to the host.
#include "common.cuh"

namespace {

template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
dyt_kernel(float* __restrict__ resid, const TY* __restrict__ y, int splits, long long split_stride, const float* __restrict__ y_bias,
           const float* __restrict__ post_w, const float* __restrict__ post_b, const float* __restrict__ post_alpha,
           float mult, const float* __restrict__ pre_w, const float* __restrict__ pre_b,
           const float* __restrict__ pre_alpha, TO* __restrict__ out, const int* __restrict__ rows, int n_out, int h,
           int write_resid) {
    qi::pdl_wait();
    const float pa = post_w ? post_alpha[0] : 0.f;
    const float al = out ? pre_alpha[0] : 0.f;
    const size_t total = (size_t)n_out * h;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t i = idx / h;
        const int c = (int)(idx % h);
        const size_t src = (rows ? (size_t)rows[i] : i) * h + c;
        float x = resid[src];
        if (y) {
            float t = qi::to_f32<TY>(y[src]);
            for (int sp = 1; sp < splits; ++sp) t += qi::to_f32<TY>(y[(size_t)sp * split_stride + src]);
            if (y_bias) t += y_bias[c];
            if (post_w) t = mult * (tanhf(pa * t) * post_w[c] + post_b[c]);
            x += t;
        }
        if (write_resid) resid[src] = x;
        if (out) out[idx] = qi::from_f32<TO>(tanhf(al * x) * pre_w[c] + pre_b[c]);
    }
}

// out[t] = [a[t] | b[t]] in the output type: the input of a projection that reads two 32-bit streams.
template <typename TO>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, TO* __restrict__ out, int n, int h) {
    qi::pdl_wait();
    const size_t total = (size_t)n * 2 * h;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / (2 * h);
        const int c = (int)(idx % (2 * h));
        out[idx] = qi::from_f32<TO>(c < h ? a[t * h + c] : b[t * h + c - h]);
    }
}

unsigned blocks_for(size_t total) {
    size_t blocks = (total + 255) / 256;
    return (unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks);
}

}  // namespace

// resid float32 [n, h] (rows picked by `rows` when given); y [n, h] in y_dtype (or `splits` such arrays, `split_stride`
// elements apart) or null; y_bias float32 [h] or null;
// post_w / post_b float32 [h] and post_alpha float32 [1] or all null (then y is added as it is); pre_* likewise with
// out [n_out, h] in out_dtype, or all null with out null.
extern "C" int qi_dyt(float* resid, const void* y, int y_dtype, int splits, long long split_stride, const float* y_bias, const float* post_w,
                      const float* post_b, const float* post_alpha, float mult, const float* pre_w, const float* pre_b,
                      const float* pre_alpha, void* out, int out_dtype, const int* rows, int n_out, int h,
                      int write_resid, cudaStream_t stream) {
    QI_REQUIRE(n_out >= 0 && h > 0, "dyt: bad sizes n=%d h=%d", n_out, h);
    QI_REQUIRE(resid, "dyt: the residual stream is missing");
    QI_REQUIRE((post_w == nullptr) == (post_b == nullptr) && (post_w == nullptr) == (post_alpha == nullptr), "dyt: a post-norm needs w, b and alpha");
    QI_REQUIRE(!post_w || y, "dyt: a post-norm without an input");
    QI_REQUIRE((out == nullptr) == (pre_w == nullptr) && (out == nullptr) == (pre_b == nullptr) && (out == nullptr) == (pre_alpha == nullptr),
               "dyt: a pre-norm needs w, b, alpha and an output");
    QI_REQUIRE(!(rows && write_resid), "dyt: picked rows do not write the stream");
    if (n_out == 0) return 0;
    const dim3 grid(blocks_for((size_t)n_out * h)), block(256);
    QI_DISPATCH_DTYPE(y ? y_dtype : qi::kF32, TY, {
        QI_DISPATCH_DTYPE(out ? out_dtype : qi::kF32, TO, {
            qi::launch(dyt_kernel<TY, TO>, grid, block, 0, stream, resid, (const TY*)y, splits, split_stride, y_bias, post_w, post_b, post_alpha, mult,
                       pre_w, pre_b, pre_alpha, (TO*)out, rows, n_out, h, write_resid);
        });
    });
    return qi::check_launch("dyt");
}

extern "C" int qi_concat_cast(const float* a, const float* b, void* out, int out_dtype, int n, int h, cudaStream_t stream) {
    QI_REQUIRE(n >= 0 && h > 0 && a && b && out, "concat_cast: bad arguments");
    if (n == 0) return 0;
    QI_DISPATCH_DTYPE(out_dtype, TO, {
        qi::launch(concat_cast_kernel<TO>, dim3(blocks_for((size_t)n * 2 * h)), dim3(256), 0, stream, a, b, (TO*)out, n, h);
    });
    return qi::check_launch("concat_cast");
}
