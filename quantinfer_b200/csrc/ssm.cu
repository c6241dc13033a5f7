// A selective state-space recurrence with one decay a head (the "state-space duality" form), and the
// gated norm that follows it.
//
// Per head h of P channels with a state S of N x P numbers (32-bit, a request's state of fixed size):
//
//     dt_t = softplus(raw_t + dt_bias_h)                      a_t = exp(-exp(A_log_h) * dt_t)
//     S_t  = a_t * S_(t-1) + dt_t * B_t x_t^T                 y_t = S_t^T C_t + D_h * x_t
//
// B_t and C_t (N numbers each) belong to the head's group (head / (heads / groups)); x, B and C are the
// outputs of the input convolution, raw_t a column of the input projection. Decays, step sizes, the state
// and all sums are 32-bit; x, B, C and raw may be bfloat16.
//
// ssm_scan: one warp walks the tokens of one step entry for `kCols` channels of one head: lane l keeps
// S[n, p] for n = l, l + 32, ... in registers, so a token costs each lane a few multiply-adds and one
// warp sum per channel; the next token's operands are requested before the current one is worked on.
// The state is read once at the entry's first token (zeros at position 0, whatever the slot holds) and
// written once after its last, so one launch serves prompts, portions and single decode tokens alike.
// State layout per slot: [heads, P, N] (N fastest, so a warp's loads are contiguous).
//
// gated_group_rmsnorm: v = y * silu(z); every `width / groups` coordinates are divided by their own root
// mean square (eps inside the root) and multiplied by a gain; 32-bit throughout, output in the activation type.
#include "common.cuh"

namespace {

constexpr int kCols = 4;       // channels a warp
constexpr int kWarps = 4;      // warps a block

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename T, int R>
__global__ void __launch_bounds__(kWarps * 32)
ssm_scan_kernel(const T* __restrict__ xbc, long long ldx, const T* __restrict__ raw_dt, long long lddt,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ state, long long state_stride, float* __restrict__ y,
                const int* __restrict__ q_start, const int* __restrict__ start_pos, const int* __restrict__ slot_ids,
                int heads, int groups, int P, int N) {
    qi::pdl_wait();
    const int h = blockIdx.x, e = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = (blockIdx.z * kWarps + warp) * kCols;
    if (p0 >= P) return;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const int t0 = q_start[e], t1 = q_start[e + 1];
    const float A = -expf(a_log[h]), bias = dt_bias[h], D = d_skip[h];
    float* st = state + (size_t)slot_ids[e] * state_stride + ((size_t)h * P + p0) * N;

    float S[kCols][R];
    const bool fresh = start_pos[e] == 0;
#pragma unroll
    for (int c = 0; c < kCols; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = lane + 32 * r;
            S[c][r] = (!fresh && n < N && p0 + c < P) ? st[(size_t)c * N + n] : 0.f;
        }

    const size_t xoff = (size_t)h * P + p0, boff = (size_t)inner + (size_t)g * N, coff = (size_t)inner + (size_t)groups * N + (size_t)g * N;
    float Bn[R], Cn[R], xn[kCols], rn;
    auto fetch = [&](int t) {
        const T* row = xbc + (size_t)t * ldx;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = lane + 32 * r;
            Bn[r] = n < N ? qi::to_f32<T>(row[boff + n]) : 0.f;
            Cn[r] = n < N ? qi::to_f32<T>(row[coff + n]) : 0.f;
        }
#pragma unroll
        for (int c = 0; c < kCols; ++c) xn[c] = p0 + c < P ? qi::to_f32<T>(row[xoff + c]) : 0.f;
        rn = qi::to_f32<T>(raw_dt[(size_t)t * lddt + h]);
    };
    if (t0 < t1) fetch(t0);
    for (int t = t0; t < t1; ++t) {
        float B[R], C[R], x[kCols];
#pragma unroll
        for (int r = 0; r < R; ++r) { B[r] = Bn[r]; C[r] = Cn[r]; }
#pragma unroll
        for (int c = 0; c < kCols; ++c) x[c] = xn[c];
        const float raw = rn;
        if (t + 1 < t1) fetch(t + 1);
        const float dt = softplus_f(raw + bias);
        const float a = expf(A * dt);
        float out[kCols];
#pragma unroll
        for (int c = 0; c < kCols; ++c) {
            const float dx = dt * x[c];
            float part = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                S[c][r] = fmaf(a, S[c][r], dx * B[r]);
                part = fmaf(S[c][r], C[r], part);
            }
            out[c] = qi::warp_sum(part) + D * x[c];
        }
        if (lane < kCols && p0 + lane < P) {
            float v = out[0];
#pragma unroll
            for (int c = 1; c < kCols; ++c) if (lane == c) v = out[c];
            y[(size_t)t * inner + xoff + lane] = v;
        }
    }
#pragma unroll
    for (int c = 0; c < kCols; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int n = lane + 32 * r;
            if (n < N && p0 + c < P) st[(size_t)c * N + n] = S[c][r];
        }
}

template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
gated_group_rmsnorm_kernel(const float* __restrict__ y, const TZ* __restrict__ z, long long ldz, const float* __restrict__ gain,
                           float eps, TO* __restrict__ out, int width, int groups) {
    __shared__ float scratch[32];
    qi::pdl_wait();
    const int t = blockIdx.x, grp = blockIdx.y;
    const int gw = width / groups;
    const float* yr = y + (size_t)t * width + (size_t)grp * gw;
    const TZ* zr = z + (size_t)t * ldz + (size_t)grp * gw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gw; i += blockDim.x) {
        const float zz = qi::to_f32<TZ>(zr[i]);
        const float v = yr[i] * (zz / (1.0f + expf(-zz)));
        ss = fmaf(v, v, ss);
    }
    const float total = qi::block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)gw + eps);
    for (int i = threadIdx.x; i < gw; i += blockDim.x) {
        const float zz = qi::to_f32<TZ>(zr[i]);
        const float v = yr[i] * (zz / (1.0f + expf(-zz)));
        out[(size_t)t * width + (size_t)grp * gw + i] = qi::from_f32<TO>(v * inv * gain[(size_t)grp * gw + i]);
    }
}

}  // namespace

// xbc [n, >= heads P + 2 groups N] in `dtype` (x | B | C, `ldx` elements a row); raw_dt [n, >= heads] in `dtype`, column h
// at raw_dt[t * lddt + h]; dt_bias, a_log, d_skip float32 [heads]; state float32, `state_stride` floats from slot to slot,
// [heads, P, N] in a slot; y float32 [n, heads P]; q_start [entries + 1], start_pos, slot_ids [entries].
extern "C" int qi_ssm_scan(const void* xbc, long long ldx, const void* raw_dt, long long lddt, int dtype, const float* dt_bias,
                           const float* a_log, const float* d_skip, float* state, long long state_stride, float* y,
                           const int* q_start, const int* start_pos, const int* slot_ids, int n_entries, int heads,
                           int groups, int P, int N, cudaStream_t stream) {
    QI_REQUIRE(n_entries >= 0 && heads > 0 && groups > 0 && P > 0 && N > 0, "ssm_scan: bad sizes");
    QI_REQUIRE(heads % groups == 0, "ssm_scan: %d heads are not a multiple of %d groups", heads, groups);
    QI_REQUIRE(N <= 256, "ssm_scan: a state of %d rows is above this kernel's 256", N);
    QI_REQUIRE(ldx >= (long long)heads * P + 2ll * groups * N && lddt >= heads, "ssm_scan: the rows are too short");
    QI_REQUIRE(state_stride >= (long long)heads * P * N, "ssm_scan: the slots of the state overlap");
    QI_REQUIRE(heads <= 0x7fffffff && n_entries <= 65535, "ssm_scan: grid too large");
    if (n_entries == 0) return 0;
    const dim3 grid(heads, n_entries, (P + kWarps * kCols - 1) / (kWarps * kCols)), block(kWarps * 32);
    const int R = (N + 31) / 32;
#define QI_SCAN(RR)                                                                                                         \
    QI_DISPATCH_DTYPE(dtype, T, {                                                                                           \
        qi::launch(ssm_scan_kernel<T, RR>, grid, block, 0, stream, (const T*)xbc, ldx, (const T*)raw_dt, lddt, dt_bias,     \
                   a_log, d_skip, state, state_stride, y, q_start, start_pos, slot_ids, heads, groups, P, N);               \
    })
    if (R <= 1) QI_SCAN(1);
    else if (R <= 2) QI_SCAN(2);
    else if (R <= 4) QI_SCAN(4);
    else QI_SCAN(8);
#undef QI_SCAN
    return qi::check_launch("ssm_scan");
}

// y float32 [n, width]; z [n, >= width] in z_dtype with `ldz` elements a row; gain float32 [width]; out [n, width] in out_dtype.
extern "C" int qi_gated_group_rmsnorm(const float* y, const void* z, int z_dtype, long long ldz, const float* gain, float eps,
                                      void* out, int out_dtype, int n, int width, int groups, cudaStream_t stream) {
    QI_REQUIRE(n >= 0 && width > 0 && groups > 0 && width % groups == 0, "gated_group_rmsnorm: bad sizes n=%d width=%d groups=%d", n, width, groups);
    QI_REQUIRE(ldz >= width && groups <= 65535, "gated_group_rmsnorm: bad layout");
    if (n == 0) return 0;
    QI_DISPATCH_DTYPE(z_dtype, TZ, {
        QI_DISPATCH_DTYPE(out_dtype, TO, {
            qi::launch(gated_group_rmsnorm_kernel<TZ, TO>, dim3(n, groups), dim3(256), 0, stream, y, (const TZ*)z, ldz, gain, eps,
                       (TO*)out, width, groups);
        });
    });
    return qi::check_launch("gated_group_rmsnorm");
}
