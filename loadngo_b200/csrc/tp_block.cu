// The pieces of gpt-oss's attention block around the attention itself, in bf16, for the
// tensor-parallel layout (one KV group per GPU): RMSNorm, the QKV and output projections, the
// residual add, and the one collective of the block, the all-reduce after the row-parallel output
// projection.
//
// Reference arithmetic: `rms_norm` gpt-oss/src/model.rs:274-280 (kernel rmsnorm_rows,
// metal-compute/src/kernels.metal:1096-1117); projections `layer.q/k/v/o.mul_vec` + `add`
// model.rs:424-429, 465-467 with bf16 weights as weights/src/dense.rs:82-94 (row . x, widened
// exactly, one rounding at the end); `add_rows` kernels.metal:1648-1659.  The reference has no
// collective at all: the all-reduce exists because the heads are split over GPUs here.
//
// The projections are plain dense GEMMs and go to cuBLASLt; the all-reduce goes to NCCL over
// NVLink.  Both libraries are opened on first use (dlopen), so the attention kernels of this
// library load and run on machines that have neither.
#include "../../include/cuda_compute.h"

#include <cublasLt.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>

#include "kernels.cuh"
#include "ptx.cuh"

namespace {

int fail(int code, const char *fmt, const char *arg = "") {
    char text[320];
    snprintf(text, sizeof text, fmt, arg);
    return cc::set_error(code, text);
}

void *open_first(std::initializer_list<const char *> names) {
    for (const char *n : names)
        if (void *h = dlopen(n, RTLD_NOW | RTLD_GLOBAL)) return h;
    return nullptr;
}

// ---- cuBLASLt, resolved at run time -------------------------------------------------------------
struct Lt {
    decltype(&cublasLtCreate) create;
    decltype(&cublasLtDestroy) destroy;
    decltype(&cublasLtMatmul) matmul;
    decltype(&cublasLtMatmulDescCreate) desc_create;
    decltype(&cublasLtMatmulDescDestroy) desc_destroy;
    decltype(&cublasLtMatmulDescSetAttribute) desc_set;
    decltype(&cublasLtMatrixLayoutCreate) layout_create;
    decltype(&cublasLtMatrixLayoutDestroy) layout_destroy;
    decltype(&cublasLtMatmulPreferenceCreate) pref_create;
    decltype(&cublasLtMatmulPreferenceDestroy) pref_destroy;
    decltype(&cublasLtMatmulPreferenceSetAttribute) pref_set;
    decltype(&cublasLtMatmulAlgoGetHeuristic) heuristic;
    bool ok = false;
};

const Lt &lt() {
    static Lt api = [] {
        Lt a{};
        void *h = open_first({"libcublasLt.so.12", "/usr/local/cuda/lib64/libcublasLt.so.12", "libcublasLt.so"});
        if (!h) return a;
#define CC_SYM(field, name) a.field = reinterpret_cast<decltype(a.field)>(dlsym(h, #name))
        CC_SYM(create, cublasLtCreate);
        CC_SYM(destroy, cublasLtDestroy);
        CC_SYM(matmul, cublasLtMatmul);
        CC_SYM(desc_create, cublasLtMatmulDescCreate);
        CC_SYM(desc_destroy, cublasLtMatmulDescDestroy);
        CC_SYM(desc_set, cublasLtMatmulDescSetAttribute);
        CC_SYM(layout_create, cublasLtMatrixLayoutCreate);
        CC_SYM(layout_destroy, cublasLtMatrixLayoutDestroy);
        CC_SYM(pref_create, cublasLtMatmulPreferenceCreate);
        CC_SYM(pref_destroy, cublasLtMatmulPreferenceDestroy);
        CC_SYM(pref_set, cublasLtMatmulPreferenceSetAttribute);
        CC_SYM(heuristic, cublasLtMatmulAlgoGetHeuristic);
#undef CC_SYM
        a.ok = a.create && a.destroy && a.matmul && a.desc_create && a.desc_destroy && a.desc_set && a.layout_create &&
               a.layout_destroy && a.pref_create && a.pref_destroy && a.pref_set && a.heuristic;
        return a;
    }();
    return api;
}

// ---- NCCL, resolved at run time -----------------------------------------------------------------
struct Nccl {
    decltype(&ncclGetUniqueId) unique_id;
    decltype(&ncclCommInitRank) init_rank;
    decltype(&ncclCommDestroy) destroy;
    decltype(&ncclAllReduce) all_reduce;
    decltype(&ncclGetErrorString) error_string;
    bool ok = false;
};

const Nccl &nccl() {
    static Nccl api = [] {
        Nccl a{};
        void *h = open_first({"libnccl.so.2", "/usr/lib/x86_64-linux-gnu/libnccl.so.2", "libnccl.so"});
        if (!h) return a;
        a.unique_id = reinterpret_cast<decltype(a.unique_id)>(dlsym(h, "ncclGetUniqueId"));
        a.init_rank = reinterpret_cast<decltype(a.init_rank)>(dlsym(h, "ncclCommInitRank"));
        a.destroy = reinterpret_cast<decltype(a.destroy)>(dlsym(h, "ncclCommDestroy"));
        a.all_reduce = reinterpret_cast<decltype(a.all_reduce)>(dlsym(h, "ncclAllReduce"));
        a.error_string = reinterpret_cast<decltype(a.error_string)>(dlsym(h, "ncclGetErrorString"));
        a.ok = a.unique_id && a.init_rank && a.destroy && a.all_reduce && a.error_string;
        return a;
    }();
    return api;
}

// ---- kernels ------------------------------------------------------------------------------------
// One warp per row: out = x * (1 / sqrt(mean(x^2) + eps)) * w, x and out bf16, w f32.  The mean
// is accumulated in f32 over f32-widened inputs (the reference uses an f64 mean; for 2880 bf16
// inputs the difference is far below the bf16 output rounding).
__global__ void __launch_bounds__(256) rmsnorm_bf16_kernel(const uint16_t *x, const float *w, uint16_t *out,
                                                           uint32_t rows, uint32_t d, float eps) {
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (row >= rows) return;
    const uint32_t *xr = reinterpret_cast<const uint32_t *>(x + static_cast<size_t>(row) * d);
    const uint32_t pairs = d / 2;
    float sum = 0.f;
    for (uint32_t i = lane; i < pairs; i += 32) {
        const uint32_t v = xr[i];
        const float a = __uint_as_float(v << 16), b = __uint_as_float(v & 0xffff0000u);
        sum += a * a + b * b;
    }
    for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float scale = 1.0f / sqrtf(sum / static_cast<float>(d) + eps);
    uint32_t *orow = reinterpret_cast<uint32_t *>(out + static_cast<size_t>(row) * d);
    const float2 *w2 = reinterpret_cast<const float2 *>(w);
    for (uint32_t i = lane; i < pairs; i += 32) {
        const uint32_t v = xr[i];
        const float2 ww = w2[i];
        const float a = __uint_as_float(v << 16) * scale * ww.x, b = __uint_as_float(v & 0xffff0000u) * scale * ww.y;
        orow[i] = cc::pack_bf16x2(a, b);
    }
}

// h[r][c] += o[r][c] (+ bias[c]), bf16 in place, two elements per thread step.
__global__ void __launch_bounds__(256) residual_add_bf16_kernel(uint16_t *h, const uint16_t *o, const float *bias,
                                                                uint64_t pairs, uint32_t width_pairs) {
    for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < pairs;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t hv = reinterpret_cast<uint32_t *>(h)[i], ov = reinterpret_cast<const uint32_t *>(o)[i];
        float a = __uint_as_float(hv << 16) + __uint_as_float(ov << 16);
        float b = __uint_as_float(hv & 0xffff0000u) + __uint_as_float(ov & 0xffff0000u);
        if (bias) {
            const uint32_t c = static_cast<uint32_t>(i % width_pairs) * 2;
            a += bias[c];
            b += bias[c + 1];
        }
        reinterpret_cast<uint32_t *>(h)[i] = cc::pack_bf16x2(a, b);
    }
}

}  // namespace

struct cc_blas {
    cublasLtHandle_t handle = nullptr;
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    std::mutex mu;
    std::map<std::tuple<uint32_t, uint32_t, uint32_t>, cublasLtMatmulAlgo_t> algos;
};

struct cc_comm {
    ncclComm_t comm = nullptr;
    int world = 1, rank = 0;
};

extern "C" int cc_blas_new(cc_blas **out) {
    if (!out) return fail(CC_DISPATCH, "blas: null output");
    if (!lt().ok) return fail(CC_COMPILE, "cuBLASLt could not be opened (libcublasLt.so.12)");
    cc_blas *b = new cc_blas;
    if (lt().create(&b->handle) != CUBLAS_STATUS_SUCCESS) {
        delete b;
        return fail(CC_GPU, "cublasLtCreate failed");
    }
    b->workspace_bytes = 64u << 20;
    if (cudaMalloc(&b->workspace, b->workspace_bytes) != cudaSuccess) {
        cudaGetLastError();
        lt().destroy(b->handle);
        delete b;
        return fail(CC_ALLOC, "could not allocate the 64 MiB GEMM workspace");
    }
    *out = b;
    return CC_OK;
}

extern "C" void cc_blas_free(cc_blas *b) {
    if (!b) return;
    cudaFree(b->workspace);
    lt().destroy(b->handle);
    delete b;
}

extern "C" int cc_gemm_bf16(cc_blas *b, void *stream, const void *a, const void *w, void *out, uint32_t m,
                            uint32_t n, uint32_t k, uint32_t lda, uint32_t ldw, uint32_t ldo) {
    if (!b || !a || !w || !out) return fail(CC_DISPATCH, "gemm: null argument");
    if (m == 0 || n == 0 || k == 0 || lda < k || ldw < k || ldo < n) return fail(CC_DISPATCH, "gemm: bad shape or stride");
    const Lt &L = lt();
    // Row-major out[m][n] = a[m][k] . w[n][k]^T is, column-major, out^T (n x m) = w^T . a.
    cublasLtMatmulDesc_t desc = nullptr;
    cublasLtMatrixLayout_t lw = nullptr, la = nullptr, lo = nullptr;
    cublasLtMatmulPreference_t pref = nullptr;
    int rc = CC_OK;
    const cublasOperation_t tr = CUBLAS_OP_T, no = CUBLAS_OP_N;
    const float one = 1.0f, zero = 0.0f;
    bool good = L.desc_create(&desc, CUBLAS_COMPUTE_32F, CUDA_R_32F) == CUBLAS_STATUS_SUCCESS &&
                L.desc_set(desc, CUBLASLT_MATMUL_DESC_TRANSA, &tr, sizeof tr) == CUBLAS_STATUS_SUCCESS &&
                L.desc_set(desc, CUBLASLT_MATMUL_DESC_TRANSB, &no, sizeof no) == CUBLAS_STATUS_SUCCESS &&
                L.layout_create(&lw, CUDA_R_16BF, k, n, ldw) == CUBLAS_STATUS_SUCCESS &&
                L.layout_create(&la, CUDA_R_16BF, k, m, lda) == CUBLAS_STATUS_SUCCESS &&
                L.layout_create(&lo, CUDA_R_16BF, n, m, ldo) == CUBLAS_STATUS_SUCCESS;
    if (good) {
        std::lock_guard<std::mutex> lock(b->mu);
        const auto key = std::make_tuple(m, n, k);
        auto it = b->algos.find(key);
        if (it == b->algos.end()) {
            cublasLtMatmulHeuristicResult_t result{};
            int found = 0;
            good = L.pref_create(&pref) == CUBLAS_STATUS_SUCCESS &&
                   L.pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &b->workspace_bytes,
                              sizeof b->workspace_bytes) == CUBLAS_STATUS_SUCCESS &&
                   L.heuristic(b->handle, desc, lw, la, lo, lo, pref, 1, &result, &found) == CUBLAS_STATUS_SUCCESS &&
                   found > 0;
            if (good) it = b->algos.emplace(key, result.algo).first;
        }
        if (good) {
            const cublasStatus_t st = L.matmul(b->handle, desc, &one, w, lw, a, la, &zero, out, lo, out, lo, &it->second,
                                               b->workspace, b->workspace_bytes, static_cast<cudaStream_t>(stream));
            if (st != CUBLAS_STATUS_SUCCESS) rc = fail(CC_GPU, "cublasLtMatmul failed");
        }
    }
    if (!good && rc == CC_OK) rc = fail(CC_GPU, "cuBLASLt could not set this GEMM up");
    if (pref) L.pref_destroy(pref);
    if (lo) L.layout_destroy(lo);
    if (la) L.layout_destroy(la);
    if (lw) L.layout_destroy(lw);
    if (desc) L.desc_destroy(desc);
    return rc;
}

extern "C" int cc_rmsnorm_bf16(void *stream, const void *x, const float *w, void *out, uint32_t rows, uint32_t d,
                               float eps) {
    if (!x || !w || !out) return fail(CC_DISPATCH, "rmsnorm: null argument");
    if (rows == 0 || d == 0 || d % 2 != 0) return fail(CC_DISPATCH, "rmsnorm: unsupported rows (width must be even)");
    rmsnorm_bf16_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t *>(x), w, static_cast<uint16_t *>(out), rows, d, eps);
    return cudaGetLastError() == cudaSuccess ? CC_OK : fail(CC_GPU, "rmsnorm launch failed");
}

extern "C" int cc_residual_add_bf16(void *stream, void *h, const void *o, const float *bias, uint32_t rows,
                                    uint32_t width) {
    if (!h || !o) return fail(CC_DISPATCH, "residual_add: null argument");
    if (rows == 0 || width == 0 || width % 2 != 0) return fail(CC_DISPATCH, "residual_add: unsupported shape");
    const uint64_t pairs = static_cast<uint64_t>(rows) * width / 2;
    uint64_t blocks = (pairs + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    residual_add_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint16_t *>(h), static_cast<const uint16_t *>(o), bias, pairs, width / 2);
    return cudaGetLastError() == cudaSuccess ? CC_OK : fail(CC_GPU, "residual_add launch failed");
}

extern "C" int cc_comm_unique_id(void *id128) {
    if (!id128) return fail(CC_DISPATCH, "comm: null id");
    if (!nccl().ok) return fail(CC_COMPILE, "NCCL could not be opened (libnccl.so.2)");
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    const ncclResult_t r = nccl().unique_id(static_cast<ncclUniqueId *>(id128));
    return r == ncclSuccess ? CC_OK : fail(CC_GPU, "ncclGetUniqueId: %s", nccl().error_string(r));
}

extern "C" int cc_comm_init(const void *id128, int world, int rank, cc_comm **out) {
    if (!id128 || !out || world < 1 || rank < 0 || rank >= world) return fail(CC_DISPATCH, "comm: bad arguments");
    if (!nccl().ok) return fail(CC_COMPILE, "NCCL could not be opened (libnccl.so.2)");
    cc_comm *c = new cc_comm;
    c->world = world;
    c->rank = rank;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    const ncclResult_t r = nccl().init_rank(&c->comm, world, id, rank);
    if (r != ncclSuccess) {
        delete c;
        return fail(CC_GPU, "ncclCommInitRank: %s", nccl().error_string(r));
    }
    *out = c;
    return CC_OK;
}

extern "C" void cc_comm_free(cc_comm *c) {
    if (!c) return;
    if (c->comm) nccl().destroy(c->comm);
    delete c;
}

extern "C" int cc_all_reduce_bf16(cc_comm *c, void *stream, void *buffer, size_t count) {
    if (!c || !buffer) return fail(CC_DISPATCH, "all_reduce: null argument");
    if (count == 0) return CC_OK;
    const ncclResult_t r = nccl().all_reduce(buffer, buffer, count, ncclBfloat16, ncclSum, c->comm,
                                             static_cast<cudaStream_t>(stream));
    return r == ncclSuccess ? CC_OK : fail(CC_GPU, "ncclAllReduce: %s", nccl().error_string(r));
}
