// Fused YaRN-RoPE + paged bf16 KV append.
//
// Replaces, for the new positions of one layer, the three calls loadngo's GPU forward pass
// makes through metal-compute (gpt-oss/src/gpu.rs:741-759): `rotate_halves` on Q,
// `rotate_halves` on K, and the `copy_rows` pair that puts the new K and V rows into the
// cache.  The arithmetic is that of the CPU reference (gpt-oss/src/model.rs:389-404): element
// i of a head's first half turns with element i of its second, `a*c - b*s` and `b*c + a*s`
// in f32 with separately rounded products (no fused multiply-add), against a (cos, sin)
// table the host computed in f64 and cast to f32 (gpt-oss/src/gpu.rs:689-697).
//
// Outputs: rotated Q as two bf16 planes hi + lo (hi = bf16(q), lo = bf16(q - hi)), which
// keeps 16 mantissa bits for the attention kernels without an f32 round trip; rotated K
// and raw V rounded to bf16 (nearest even, weights/src/dtype.rs:102-110) straight into
// their page.  HBM-bound: each element is read once and written once.
#include "kernels.cuh"
#include "ptx.cuh"

namespace cc {
namespace {

template <bool F32>
__device__ __forceinline__ void load8(const void *base, size_t elem, float (&out)[8]) {
    if constexpr (F32) {
        const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem);
        float4 x = p[0], y = p[1];
        out[0] = x.x; out[1] = x.y; out[2] = x.z; out[3] = x.w;
        out[4] = y.x; out[5] = y.y; out[6] = y.z; out[7] = y.w;
    } else {
        uint4 raw = *reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(base) + elem);
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            out[2 * j] = __uint_as_float(w[j] << 16);
            out[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
    return make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]),
                      pack_bf16x2(x[6], x[7]));
}

// Rotates 8 pairs (first-half elements a, second-half elements b) by table entries cs.
__device__ __forceinline__ void rotate8(float (&a)[8], float (&b)[8], const float *cs) {
    const float4 *t = reinterpret_cast<const float4 *>(cs);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float4 e = t[j];  // cos, sin, cos, sin
        float a0 = a[2 * j], b0 = b[2 * j], a1 = a[2 * j + 1], b1 = b[2 * j + 1];
        a[2 * j] = __fsub_rn(__fmul_rn(a0, e.x), __fmul_rn(b0, e.y));
        b[2 * j] = __fadd_rn(__fmul_rn(b0, e.x), __fmul_rn(a0, e.y));
        a[2 * j + 1] = __fsub_rn(__fmul_rn(a1, e.z), __fmul_rn(b1, e.w));
        b[2 * j + 1] = __fadd_rn(__fmul_rn(b1, e.z), __fmul_rn(a1, e.w));
    }
}

template <bool F32>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeAppendParams p) {
    const uint32_t q_items = p.heads * 4, k_items = p.kv_heads * 4, v_items = p.kv_heads * 8;
    const uint32_t per_token = q_items + k_items + v_items;
    const uint64_t total = static_cast<uint64_t>(p.n) * per_token;
    for (uint64_t item = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; item < total;
         item += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t token = static_cast<uint32_t>(item / per_token);
        uint32_t j = static_cast<uint32_t>(item % per_token);
        const int64_t pos = p.positions[token];
        const int64_t row = pos - p.table_start;
        if (pos < 0 || row < 0 || row >= p.table_rows) {
            raise_status(p.status, kStatusBadTableRow);
            continue;
        }
        const float *cs_row = p.table + row * (kHeadDim / 2) * 2;
        if (j < q_items) {
            const uint32_t head = j >> 2, c = j & 3;
            const size_t base = (static_cast<size_t>(token) * p.heads + head) * kHeadDim + c * 8;   // q_hi / q_lo rows
            const size_t src = static_cast<size_t>(token) * p.q_stride + head * kHeadDim + c * 8;
            float a[8], b[8];
            load8<F32>(p.q, src, a);
            load8<F32>(p.q, src + 32, b);
            rotate8(a, b, cs_row + c * 16);
            uint4 ha = pack8(a), hb = pack8(b);
            *reinterpret_cast<uint4 *>(p.q_hi + base) = ha;
            *reinterpret_cast<uint4 *>(p.q_hi + base + 32) = hb;
            if (p.q_lo) {
                float la[8], lb[8];
                const uint32_t wa[4] = {ha.x, ha.y, ha.z, ha.w}, wb[4] = {hb.x, hb.y, hb.z, hb.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    la[2 * e] = a[2 * e] - __uint_as_float(wa[e] << 16);
                    la[2 * e + 1] = a[2 * e + 1] - __uint_as_float(wa[e] & 0xffff0000u);
                    lb[2 * e] = b[2 * e] - __uint_as_float(wb[e] << 16);
                    lb[2 * e + 1] = b[2 * e + 1] - __uint_as_float(wb[e] & 0xffff0000u);
                }
                *reinterpret_cast<uint4 *>(p.q_lo + base) = pack8(la);
                *reinterpret_cast<uint4 *>(p.q_lo + base + 32) = pack8(lb);
            }
            continue;
        }
        // K and V go to the token's page.
        const uint32_t seq = static_cast<uint32_t>(p.seq_ids[token]);
        uint32_t logical = static_cast<uint32_t>(pos / kPageTokens);
        if (p.ring_pages) logical %= p.ring_pages;
        if (logical >= p.max_pages) {
            raise_status(p.status, kStatusBadPage);
            continue;
        }
        const int32_t page = p.block_table[static_cast<size_t>(seq) * p.max_pages + logical];
        if (page < 0 || static_cast<uint32_t>(page) >= p.pool_pages) {
            raise_status(p.status, kStatusBadPage);
            continue;
        }
        const uint32_t slot = static_cast<uint32_t>(pos % kPageTokens);
        j -= q_items;
        if (j < k_items) {
            const uint32_t head = j >> 2, c = j & 3;
            const size_t base = static_cast<size_t>(token) * p.k_stride + head * kHeadDim + c * 8;
            float a[8], b[8];
            load8<F32>(p.k, base, a);
            load8<F32>(p.k, base + 32, b);
            rotate8(a, b, cs_row + c * 16);
            uint16_t *dst = p.pool + ((static_cast<size_t>(page) * p.kv_heads + head) * kTileRows + slot) * kHeadDim +
                            c * 8;
            *reinterpret_cast<uint4 *>(dst) = pack8(a);
            *reinterpret_cast<uint4 *>(dst + 32) = pack8(b);
        } else {
            j -= k_items;
            const uint32_t head = j >> 3, c = j & 7;
            const size_t base = static_cast<size_t>(token) * p.v_stride + head * kHeadDim + c * 8;
            float x[8];
            load8<F32>(p.v, base, x);
            uint16_t *dst = p.pool +
                            ((static_cast<size_t>(page) * p.kv_heads + head) * kTileRows + kPageTokens + slot) *
                                kHeadDim +
                            c * 8;
            *reinterpret_cast<uint4 *>(dst) = pack8(x);
        }
    }
}

}  // namespace

void launch_rope_append(const RopeAppendParams &p, cudaStream_t stream) {
    const uint64_t per_token = p.heads * 4ull + p.kv_heads * 12ull;
    const uint64_t total = p.n * per_token;
    if (total == 0) return;
    uint64_t blocks = (total + 255) / 256;
    const uint64_t cap = 148ull * 8 * 4;  // a few waves of the 148 SMs; the loop strides beyond
    if (blocks > cap) blocks = cap;
    if (p.in_f32)
        rope_append_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    else
        rope_append_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
}

}  // namespace cc
