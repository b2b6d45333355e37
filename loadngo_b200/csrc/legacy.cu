// The float32 entry points of metal-compute's Batch that gpt-oss's attention phase uses, with
// their original shapes and semantics (ring of `slots` rows, f32 activations): copy_rows,
// add_rows, rmsnorm_rows, rotate_halves and grouped attention.  They keep an unmodified caller
// working; the fast path is the paged bf16 one (rope_append.cu, decode.cu, prefill.cu).
//
// Semantics follow metal-compute/src/kernels.metal: rmsnorm_rows 1096-1117, copy_rows
// 1127-1138, add_rows 1648-1659, rotate_halves 1672-1690, attention_grouped 500-577 /
// attention_grouped_narrow 1944-2032.
#include "legacy.cuh"

namespace cc {
namespace {

__global__ void copy_rows_kernel(const float *src, float *dst, uint32_t rows, uint32_t width, uint32_t src_stride,
                                 uint32_t dst_stride) {
    const uint64_t n = static_cast<uint64_t>(rows) * width;
    for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint64_t r = i / width, c = i % width;
        dst[r * dst_stride + c] = src[r * src_stride + c];
    }
}

__global__ void add_rows_kernel(float *dst, const float *src, uint32_t rows, uint32_t width, uint32_t src_stride) {
    const uint64_t n = static_cast<uint64_t>(rows) * width;
    for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint64_t r = i / width, c = i % width;
        dst[i] = __fadd_rn(dst[i], src[r * src_stride + c]);
    }
}

// One warp per row: v = w * v / sqrt(mean(v^2) + eps).
__global__ void rmsnorm_rows_kernel(float *v, const float *w, uint32_t rows, uint32_t d, uint32_t stride, float eps) {
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (row >= rows) return;
    float *x = v + static_cast<uint64_t>(row) * stride;
    float sum = 0.f;
    for (uint32_t i = lane; i < d; i += 32) sum += x[i] * x[i];
    for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float scale = 1.0f / sqrtf(sum / static_cast<float>(d) + eps);
    for (uint32_t i = lane; i < d; i += 32) x[i] = x[i] * scale * w[i];
}

// x [rows][heads][dim], table [rows][rotary/2] (cos, sin): element i of the first half of the
// rotated part turns with element i of its second half.
__global__ void rotate_halves_kernel(float *x, const float2 *table, uint32_t rows, uint32_t heads, uint32_t dim,
                                     uint32_t rotary) {
    const uint32_t half = rotary / 2;
    const uint64_t n = static_cast<uint64_t>(rows) * heads * half;
    for (uint64_t idx = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; idx < n;
         idx += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t i = idx % half;
        const uint64_t rh = idx / half;  // row * heads + head
        const uint64_t row = rh / heads;
        const float2 cs = table[row * half + i];
        float *head = x + rh * dim;
        const float a = head[i], b = head[i + half];
        head[i] = __fsub_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y));
        head[i + half] = __fadd_rn(__fmul_rn(b, cs.x), __fmul_rn(a, cs.y));
    }
}

// Grouped attention, one CTA per (new position, query head); 4 warps walk interleaved keys,
// each lane owning dim/32 value columns; partials merge in shared memory with the sink.
constexpr int kAttnWarps = 4;
constexpr int kMaxPerLane = 16;  // dim <= 512

__global__ void __launch_bounds__(kAttnWarps * 32) attention_grouped_kernel(const float *q, const float *k,
                                                                           const float *v, float *out,
                                                                           const float *sinks, GroupedArgs a) {
    __shared__ float part_m[kAttnWarps], part_l[kAttnWarps];
    extern __shared__ float part_acc[];  // [kAttnWarps][dim]
    const uint32_t step = blockIdx.x / a.heads, head = blockIdx.x % a.heads;
    const uint32_t kv = head / (a.heads / a.kv_heads);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t per = a.dim / 32;
    const float *qt = q + (static_cast<uint64_t>(step) * a.heads + head) * a.dim;
    float qr[kMaxPerLane], acc[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        qr[i] = static_cast<uint32_t>(i) < per ? qt[lane + 32 * i] : 0.f;
        acc[i] = 0.f;
    }
    const uint32_t last = a.start + step;
    const uint32_t first = last + 1 > a.window ? last + 1 - a.window : 0;
    const uint64_t row = static_cast<uint64_t>(a.kv_heads) * a.dim;
    const uint64_t at = static_cast<uint64_t>(kv) * a.dim;
    float m = -INFINITY, l = 0.f;
    for (uint32_t s = first + warp; s <= last; s += kAttnWarps) {
        const float *kr = k + static_cast<uint64_t>(s % a.slots) * row + at;
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i)
            if (static_cast<uint32_t>(i) < per) dot += qr[i] * kr[lane + 32 * i];
        for (int off = 16; off; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float score = dot * a.scale;
        const float next = fmaxf(m, score);
        const float keep = m == -INFINITY ? 0.f : expf(m - next);
        const float p = expf(score - next);
        l = l * keep + p;
        const float *vr = v + static_cast<uint64_t>(s % a.slots) * row + at;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i)
            if (static_cast<uint32_t>(i) < per) acc[i] = acc[i] * keep + p * vr[lane + 32 * i];
        m = next;
    }
    if (lane == 0) {
        part_m[warp] = m;
        part_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
        if (static_cast<uint32_t>(i) < per) part_acc[warp * a.dim + lane + 32 * i] = acc[i];
    __syncthreads();
    const float sink = a.sinks ? sinks[head] : -INFINITY;
    float total_max = sink;
    for (int g = 0; g < kAttnWarps; ++g) total_max = fmaxf(total_max, part_m[g]);
    float total = sink == -INFINITY ? 0.f : expf(sink - total_max);
    float weight[kAttnWarps];
    for (int g = 0; g < kAttnWarps; ++g) {
        weight[g] = part_m[g] == -INFINITY ? 0.f : expf(part_m[g] - total_max);
        total += part_l[g] * weight[g];
    }
    float *o = out + (static_cast<uint64_t>(step) * a.heads + head) * a.dim;
    for (uint32_t d = threadIdx.x; d < a.dim; d += blockDim.x) {
        float sum = 0.f;
        for (int g = 0; g < kAttnWarps; ++g) sum += part_acc[g * a.dim + d] * weight[g];
        o[d] = sum / total;
    }
}

unsigned blocks_for(uint64_t n, unsigned threads) {
    uint64_t b = (n + threads - 1) / threads;
    const uint64_t cap = 148ull * 16;
    return static_cast<unsigned>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

void launch_copy_rows(const float *src, float *dst, uint32_t rows, uint32_t width, uint32_t src_stride,
                      uint32_t dst_stride, cudaStream_t stream) {
    copy_rows_kernel<<<blocks_for(static_cast<uint64_t>(rows) * width, 256), 256, 0, stream>>>(src, dst, rows, width,
                                                                                               src_stride, dst_stride);
}
void launch_add_rows(float *dst, const float *src, uint32_t rows, uint32_t width, uint32_t src_stride,
                     cudaStream_t stream) {
    add_rows_kernel<<<blocks_for(static_cast<uint64_t>(rows) * width, 256), 256, 0, stream>>>(dst, src, rows, width,
                                                                                              src_stride);
}
void launch_rmsnorm_rows(float *v, const float *w, uint32_t rows, uint32_t d, uint32_t stride, float eps,
                         cudaStream_t stream) {
    rmsnorm_rows_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(v, w, rows, d, stride, eps);
}
void launch_rotate_halves(float *x, const float *table, uint32_t rows, uint32_t heads, uint32_t dim, uint32_t rotary,
                          cudaStream_t stream) {
    const uint64_t n = static_cast<uint64_t>(rows) * heads * (rotary / 2);
    rotate_halves_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(x, reinterpret_cast<const float2 *>(table), rows,
                                                                 heads, dim, rotary);
}
void launch_attention_grouped(const float *q, const float *k, const float *v, float *out, const float *sinks,
                              const GroupedArgs &a, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(kAttnWarps) * a.dim * sizeof(float);
    attention_grouped_kernel<<<a.t * a.heads, kAttnWarps * 32, smem, stream>>>(q, k, v, out, sinks, a);
}

}  // namespace cc
