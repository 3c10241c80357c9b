// Depth-weighted average of the residual stream, with the residual add before it and (optionally) the RMSNorm
// after it in the same pass.
//
// A model that averages over depth keeps every block's result: X_0 is the embedding output, X_(i+1) the result
// of block i (its input stream plus what its parts add), and what the next reader sees is
//
//   x = sum over j = 0 .. i+1 of w[j] X_j            (w: the block's own stored weights, i + 2 of them)
//
// One block of threads per token row: x_new = stream (+ delta_a) (+ delta_b) becomes X_(i+1) in the history,
// the weighted sum over the history becomes the stream, and if a norm weight is given the row is normalised
// (x / sqrt(mean(x^2) + eps) * norm_w) into `out` as well, so the next block's norm costs no launch and no
// second read of the stream. Everything is float32 but the deltas and `out`, which have the activation type.
// The history is [entries, row_capacity, width] float32; block 0 also stores its input as X_0.
#include "common.cuh"

namespace celeg_b200 {

struct DepthAverageArgs {
    float* stream;                  // [rows, width], replaced by the average
    const void* delta_a; const void* delta_b;      // activation type or null
    float* history; long long entry_stride;        // floats between two entries of the history
    const float* weights;           // [index + 2]
    int index;                      // the block whose result this is: X_(index + 1)
    const float* norm_weight; void* out; float eps; // the norm after the average (null: none)
    int width;
};

template <typename A, int kPerThread>
__global__ void depth_average_kernel(const DepthAverageArgs a) {
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const int row = blockIdx.x, width = a.width;
    const size_t at = (size_t)row * width;
    float* stream = a.stream + at;
    const A* da = a.delta_a ? static_cast<const A*>(a.delta_a) + at : nullptr;
    const A* db = a.delta_b ? static_cast<const A*>(a.delta_b) + at : nullptr;
    float* history = a.history + at;
    const int last = a.index + 1;
    const float w_last = a.weights[last];
    float kept[kPerThread];
    float sum = 0.0f;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int c = threadIdx.x + u * blockDim.x;
        if (c < width) {
            const float x_in = stream[c];
            float x = x_in;
            if (da) x += to_float(da[c]);
            if (db) x += to_float(db[c]);
            if (a.index == 0) history[c] = x_in;
            history[(size_t)last * a.entry_stride + c] = x;
            float mean = 0.0f;
            for (int j = 0; j < last; ++j)
                mean = fmaf(a.weights[j], a.index == 0 ? x_in : history[(size_t)j * a.entry_stride + c], mean);
            mean = fmaf(w_last, x, mean);
            stream[c] = mean;
            kept[u] = mean;
            sum += mean * mean;
        }
    }
    if (a.norm_weight == nullptr) return;
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)width + a.eps);
    A* out = static_cast<A*>(a.out) + at;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int c = threadIdx.x + u * blockDim.x;
        if (c < width) out[c] = from_float<A>(kept[u] * inv * a.norm_weight[c]);
    }
}

// Widths that are a multiple of 4 with 16-byte aligned rows: four neighbouring elements a thread and load.
template <typename A, int kPerThread>
__global__ void depth_average_vec4_kernel(const DepthAverageArgs a) {
    __shared__ float scratch[33];
    chain_release();
    chain_wait();
    const int row = blockIdx.x, width = a.width, quads = width >> 2;
    const size_t at = (size_t)row * width;
    float4* stream = reinterpret_cast<float4*>(a.stream + at);
    const A* da = a.delta_a ? static_cast<const A*>(a.delta_a) + at : nullptr;
    const A* db = a.delta_b ? static_cast<const A*>(a.delta_b) + at : nullptr;
    float* history = a.history + at;
    const int last = a.index + 1;
    const float w_last = a.weights[last];
    auto add_delta = [](float4& x, const A* d) {
        if (sizeof(A) == 2) {
            const uint2 raw = *reinterpret_cast<const uint2*>(d);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            x.x += lo.x; x.y += lo.y; x.z += hi.x; x.w += hi.y;
        } else {
            const float4 v = *reinterpret_cast<const float4*>(d);
            x.x += v.x; x.y += v.y; x.z += v.z; x.w += v.w;
        }
    };
    float4 kept[kPerThread];
    float sum = 0.0f;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int q = threadIdx.x + u * blockDim.x;
        if (q < quads) {
            const float4 x_in = stream[q];
            float4 x = x_in;
            if (da) add_delta(x, da + 4 * q);
            if (db) add_delta(x, db + 4 * q);
            if (a.index == 0) *reinterpret_cast<float4*>(history + 4 * q) = x_in;
            *reinterpret_cast<float4*>(history + (size_t)last * a.entry_stride + 4 * q) = x;
            float4 mean = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int j = 0; j < last; ++j) {
                const float w = a.weights[j];
                const float4 h = a.index == 0 ? x_in : *reinterpret_cast<const float4*>(history + (size_t)j * a.entry_stride + 4 * q);
                mean.x = fmaf(w, h.x, mean.x); mean.y = fmaf(w, h.y, mean.y);
                mean.z = fmaf(w, h.z, mean.z); mean.w = fmaf(w, h.w, mean.w);
            }
            mean.x = fmaf(w_last, x.x, mean.x); mean.y = fmaf(w_last, x.y, mean.y);
            mean.z = fmaf(w_last, x.z, mean.z); mean.w = fmaf(w_last, x.w, mean.w);
            stream[q] = mean;
            kept[u] = mean;
            sum += mean.x * mean.x + mean.y * mean.y + mean.z * mean.z + mean.w * mean.w;
        }
    }
    if (a.norm_weight == nullptr) return;
    sum = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(sum / (float)width + a.eps);
    A* out = static_cast<A*>(a.out) + at;
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
        const int q = threadIdx.x + u * blockDim.x;
        if (q < quads) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(a.norm_weight) + q);
            const float4 v = kept[u];
            if (sizeof(A) == 2) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * inv * w.x, v.y * inv * w.y);
                const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * inv * w.z, v.w * inv * w.w);
                uint2 raw;
                raw.x = *reinterpret_cast<const unsigned*>(&lo);
                raw.y = *reinterpret_cast<const unsigned*>(&hi);
                *reinterpret_cast<uint2*>(out + 4 * q) = raw;
            } else {
                *reinterpret_cast<float4*>(out + 4 * q) = make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w);
            }
        }
    }
}

}  // namespace celeg_b200

using namespace celeg_b200;

// stream[r] <- sum_j weights[j] X_j[r] for rows 0 .. n_rows - 1, with X_(index+1) = stream (+ deltas) stored on the way;
// norm_weight / out: the RMSNorm of the new stream rows (null: not wanted).
CELEG_API int celeg_depth_average(float* stream, const void* delta_a, const void* delta_b, float* history,
                                  long long entry_stride, const float* weights, int index, const float* norm_weight,
                                  void* out, float eps, int n_rows, int width, int act_dtype, cudaStream_t stream_id) {
    CELEG_REQUIRE(n_rows >= 0 && width > 0 && index >= 0 && entry_stride >= (long long)n_rows * width,
                  "depth_average: invalid sizes rows=%d width=%d index=%d entry_stride=%lld", n_rows, width, index,
                  entry_stride);
    CELEG_REQUIRE(width <= 1024 * 16, "depth_average: a width of %d exceeds %d", width, 1024 * 16);
    CELEG_REQUIRE(act_dtype == kFloat32 || act_dtype == kBFloat16, "depth_average: unknown dtype code %d", act_dtype);
    CELEG_REQUIRE(norm_weight == nullptr || (out != nullptr && eps > 0.0f), "depth_average: a norm needs out and eps");
    if (n_rows == 0) return 0;
    const DepthAverageArgs args = {stream, delta_a, delta_b, history, entry_stride, weights, index, norm_weight, out,
                                   eps, width};
    const bool aligned = width % 4 == 0 && entry_stride % 4 == 0 &&
                         (((size_t)stream | (size_t)delta_a | (size_t)delta_b | (size_t)history | (size_t)norm_weight |
                           (size_t)out) & 15) == 0;
    if (aligned && width <= 4 * 1024 * 4) {
        const int quads = width / 4;
        const int per = quads <= 1024 ? 1 : 4;
        int vec_threads = (quads + per - 1) / per;
        vec_threads = min(1024, max(64, (vec_threads + 31) / 32 * 32));
        if (act_dtype == kFloat32) {
            if (per == 1) launch_chained_class(kChainNorm, depth_average_vec4_kernel<float, 1>, n_rows, vec_threads, 0, stream_id, args);
            else launch_chained_class(kChainNorm, depth_average_vec4_kernel<float, 4>, n_rows, vec_threads, 0, stream_id, args);
        } else {
            if (per == 1) launch_chained_class(kChainNorm, depth_average_vec4_kernel<__nv_bfloat16, 1>, n_rows, vec_threads, 0, stream_id, args);
            else launch_chained_class(kChainNorm, depth_average_vec4_kernel<__nv_bfloat16, 4>, n_rows, vec_threads, 0, stream_id, args);
        }
        return check_launch("depth_average");
    }
    // few elements a thread: the history's loads of all of them are in flight together
    const int per_thread = width <= 1024 ? 1 : width <= 4096 ? 4 : 16;
    int threads = (width + per_thread - 1) / per_thread;
    threads = min(1024, max(64, (threads + 31) / 32 * 32));
#define CELEG_DEPTH_LAUNCH(A, P) \
    launch_chained_class(kChainNorm, depth_average_kernel<A, P>, n_rows, threads, 0, stream_id, args)
    if (act_dtype == kFloat32) {
        if (per_thread == 1) CELEG_DEPTH_LAUNCH(float, 1);
        else if (per_thread == 4) CELEG_DEPTH_LAUNCH(float, 4);
        else CELEG_DEPTH_LAUNCH(float, 16);
    } else {
        if (per_thread == 1) CELEG_DEPTH_LAUNCH(__nv_bfloat16, 1);
        else if (per_thread == 4) CELEG_DEPTH_LAUNCH(__nv_bfloat16, 4);
        else CELEG_DEPTH_LAUNCH(__nv_bfloat16, 16);
    }
#undef CELEG_DEPTH_LAUNCH
    return check_launch("depth_average");
}
