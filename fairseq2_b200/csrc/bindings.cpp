// Python bindings of the sm_100a kernels (module fairseq2_b200._C).
//
// Every entry point validates shapes/dtypes/alignment on the host, launches on
// the current CUDA stream of the tensor's device and never synchronises.

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>
#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include "attention.h"
#include "comm.h"
#include "elementwise.h"
#include "gemm_tcgen05.h"
#include "generation.h"
#include "moe.h"
#include "wav2vec2.h"

namespace {

using at::Tensor;

int num_sms(const Tensor& t) { return at::cuda::getDeviceProperties(t.get_device())->multiProcessorCount; }

cudaStream_t stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

bool is_bf16(const Tensor& t) { return t.scalar_type() == at::kBFloat16; }

bool aligned16(const Tensor& t) { return reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0; }

// Number of kernels of this extension launched so far (host-side bookkeeping
// that benchmarks use to report how much of a step runs on in-tree kernels).
int64_t g_launches = 0;
int64_t launch_count() { return g_launches; }
void reset_launch_count() { g_launches = 0; }

// ---------------------------------------------------------------- status word
// One pinned, host-mapped int per process. Kernels store a non-zero code when a
// bounded wait gives up; the host can poll it without touching the stream.
int* g_status_host = nullptr;
int* g_status_dev = nullptr;

int* status_dev_ptr() {
    if (g_status_host == nullptr) {
        TORCH_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&g_status_host), sizeof(int), cudaHostAllocMapped) ==
                        cudaSuccess,
                    "cudaHostAlloc for the kernel status word failed");
        *g_status_host = 0;
        TORCH_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_status_dev), g_status_host, 0) ==
                        cudaSuccess,
                    "cudaHostGetDevicePointer for the kernel status word failed");
    }
    return g_status_dev;
}

int read_status() { return g_status_host ? *reinterpret_cast<volatile int*>(g_status_host) : 0; }

void reset_status() {
    if (g_status_host) *reinterpret_cast<volatile int*>(g_status_host) = 0;
}

void check_status() {
    const int s = read_status();
    if (s != 0) {
        reset_status();
        TORCH_CHECK(false, "a fairseq2_b200 kernel gave up on a bounded wait (code ", s & 0xff, ", site ", s >> 8, ")");
    }
}

// ----------------------------------------------------------------------- GEMM
void gemm_bf16(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, bool accumulate) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "gemm_bf16: tensors must be on a CUDA device");
    TORCH_CHECK(is_bf16(a) && is_bf16(b), "gemm_bf16: operands must be bfloat16");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm_bf16: operands must be 2-D");
    TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && out.is_contiguous(), "gemm_bf16: operands must be contiguous");
    const int64_t M = a_mn ? a.size(1) : a.size(0);
    const int64_t K = a_mn ? a.size(0) : a.size(1);
    const int64_t N = b_mn ? b.size(1) : b.size(0);
    const int64_t Kb = b_mn ? b.size(0) : b.size(1);
    TORCH_CHECK(K == Kb, "gemm_bf16: reduction dims differ (", K, " vs ", Kb, ")");
    TORCH_CHECK(out.size(0) == M && out.size(1) == N, "gemm_bf16: out must be [", M, ", ", N, "]");
    const bool f32 = out.scalar_type() == at::kFloat;
    TORCH_CHECK(f32 || is_bf16(out), "gemm_bf16: out must be bfloat16 or float32");
    TORCH_CHECK(a.size(1) % 8 == 0 && b.size(1) % 8 == 0 && N % 8 == 0,
                "gemm_bf16: row pitches must be multiples of 16 bytes");
    TORCH_CHECK(aligned16(a) && aligned16(b) && aligned16(out), "gemm_bf16: base pointers must be 16-byte aligned");
    TORCH_CHECK(M > 0 && N > 0 && K > 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31),
                "gemm_bf16: bad problem size");
    check_status();
    c10::cuda::CUDAGuard guard(a.device());
    // Tensor maps are encoded through the driver API, which needs the primary
    // context bound to the calling thread. Autograd worker threads may not have
    // issued a runtime call yet, so bind it explicitly (a no-op when current).
    TORCH_CHECK(cudaSetDevice(a.get_device()) == cudaSuccess, "gemm_bf16: cudaSetDevice failed");
    const char* err = fs2::gemm_bf16_tcgen05(a.data_ptr(), b.data_ptr(), out.data_ptr(), static_cast<int>(M),
                                             static_cast<int>(N), static_cast<int>(K), a_mn, b_mn, f32, accumulate,
                                             status_dev_ptr(), num_sms(a), stream_of(a));
    TORCH_CHECK(err == nullptr, "gemm_bf16: ", err);
    g_launches += 1;
}

// C = a[M,K] * b[N,K]^T summed over ranks and scattered by rows: rank r receives rows [r*rpr, (r+1)*rpr) of the sum
// in its fp32 [rpr, N] buffer at `out_byte_off` of its symmetric arena (`ptrs` are the arenas' base addresses).
void gemm_reduce_scatter(const Tensor& a, const Tensor& b, const std::vector<int64_t>& ptrs, int64_t out_byte_off,
                         int64_t rows_per_rank) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && is_bf16(a) && is_bf16(b) && a.dim() == 2 && b.dim() == 2 &&
                    a.is_contiguous() && b.is_contiguous() && a.size(1) == b.size(1),
                "gemm_reduce_scatter: a [M,K] and b [N,K] must be contiguous bf16 CUDA matrices");
    TORCH_CHECK(a.size(1) % 8 == 0 && aligned16(a) && aligned16(b) && out_byte_off % 16 == 0,
                "gemm_reduce_scatter: alignment");
    TORCH_CHECK(!ptrs.empty() && ptrs.size() <= 8, "gemm_reduce_scatter: between 1 and 8 ranks are supported");
    float* outs[8];
    for (size_t i = 0; i < ptrs.size(); ++i) {
        TORCH_CHECK(ptrs[i] != 0, "gemm_reduce_scatter: null peer pointer");
        outs[i] = reinterpret_cast<float*>(ptrs[i] + out_byte_off);
    }
    TORCH_CHECK(b.size(0) % 4 == 0, "gemm_reduce_scatter: N must be a multiple of 4");
    check_status();
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(cudaSetDevice(a.get_device()) == cudaSuccess, "gemm_reduce_scatter: cudaSetDevice failed");
    const char* err = fs2::gemm_reduce_scatter_bf16_tcgen05(
        a.data_ptr(), b.data_ptr(), outs, static_cast<int>(ptrs.size()), static_cast<int>(rows_per_rank),
        static_cast<int>(a.size(0)), static_cast<int>(b.size(0)), static_cast<int>(a.size(1)), status_dev_ptr(),
        num_sms(a), stream_of(a));
    TORCH_CHECK(err == nullptr, "gemm_reduce_scatter: ", err);
    g_launches += 1;
}

// GEMM over strided views of flat bf16 storage. Each operand is (storage, rows in memory, row pitch in elements);
// logical shapes: A [M, K] (or [K, M] if a_mn), B [N, K] (or [K, N] if b_mn), out [M, N] bf16/fp32.
void gemm_bf16_view(const Tensor& a, int64_t a_rows, int64_t lda, bool a_mn, const Tensor& b, int64_t b_rows, int64_t ldb,
                    bool b_mn, Tensor out, int64_t c_rows, int64_t ldc, int64_t M, int64_t N, int64_t K,
                    bool accumulate, int64_t k_splits) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda() && is_bf16(a) && is_bf16(b) && a.is_contiguous() &&
                    b.is_contiguous() && out.is_contiguous() && aligned16(a) && aligned16(b) && aligned16(out),
                "gemm_bf16_view: operands must be contiguous, 16-byte aligned CUDA storage (bf16 inputs)");
    const bool f32 = out.scalar_type() == at::kFloat;
    TORCH_CHECK(f32 || is_bf16(out), "gemm_bf16_view: out must be bfloat16 or float32");
    const int64_t a_cols = a_mn ? M : K, b_cols = b_mn ? N : K;
    const int64_t esz_c = f32 ? 4 : 2;
    TORCH_CHECK(M > 0 && N > 0 && K > 0 && lda > 0 && ldb > 0 && ldc > 0 && a_rows > 0 && b_rows > 0 && c_rows > 0,
                "gemm_bf16_view: sizes must be positive");
    TORCH_CHECK((lda * 2) % 16 == 0 && (ldb * 2) % 16 == 0 && (ldc * esz_c) % 16 == 0 &&
                    ((a_mn && b_mn) || K % 8 == 0) && (a_mn ? M % 8 == 0 : true) && (b_mn ? N % 8 == 0 : true) && (N * esz_c) % 16 == 0,
                "gemm_bf16_view: row pitches and row lengths must be multiples of 16 bytes");
    TORCH_CHECK((a_rows - 1) * lda + a_cols <= a.numel() && (b_rows - 1) * ldb + b_cols <= b.numel() &&
                    (c_rows - 1) * ldc + N <= out.numel(),
                "gemm_bf16_view: a view reaches beyond its storage");
    check_status();
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(cudaSetDevice(a.get_device()) == cudaSuccess, "gemm_bf16_view: cudaSetDevice failed");
    const char* err = fs2::gemm_bf16_tcgen05_view(a.data_ptr(), lda, a_rows, b.data_ptr(), ldb, b_rows, out.data_ptr(), ldc,
                                                  c_rows, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                                                  a_mn, b_mn, f32, accumulate, status_dev_ptr(), num_sms(a), stream_of(a),
                                                  static_cast<int>(k_splits));
    TORCH_CHECK(err == nullptr, "gemm_bf16_view: ", err);
    g_launches += 1;
}

// bf16 scatter form of the fused row-parallel GEMM: tile rows owned by rank r land in slice `rank` of the
// [world, rows_per_rank, N] bf16 buffer at `slices_byte_off` of rank r's arena.
void gemm_scatter(const Tensor& a, const Tensor& b, const std::vector<int64_t>& ptrs, int64_t rank,
                  int64_t slices_byte_off, int64_t rows_per_rank, bool b_mn) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && is_bf16(a) && is_bf16(b) && a.dim() == 2 && b.dim() == 2 &&
                    a.is_contiguous() && b.is_contiguous() && a.size(1) == b.size(b_mn ? 0 : 1),
                "gemm_scatter: a [M,K] and b [N,K] (or [K,N] with b_mn) must be contiguous bf16 CUDA matrices");
    TORCH_CHECK(a.size(1) % 8 == 0 && b.size(0) % 8 == 0 && b.size(1) % 8 == 0 && aligned16(a) && aligned16(b) &&
                    slices_byte_off % 16 == 0,
                "gemm_scatter: alignment");
    TORCH_CHECK(!ptrs.empty() && ptrs.size() <= 8 && rank >= 0 && rank < static_cast<int64_t>(ptrs.size()),
                "gemm_scatter: between 1 and 8 ranks are supported");
    void* outs[8];
    for (size_t i = 0; i < ptrs.size(); ++i) {
        TORCH_CHECK(ptrs[i] != 0, "gemm_scatter: null peer pointer");
        outs[i] = reinterpret_cast<void*>(ptrs[i] + slices_byte_off);
    }
    check_status();
    c10::cuda::CUDAGuard guard(a.device());
    const char* err = fs2::gemm_scatter_bf16_tcgen05(
        a.data_ptr(), b.data_ptr(), b_mn, outs, static_cast<int>(ptrs.size()), static_cast<int>(rank),
        static_cast<int>(rows_per_rank), static_cast<int>(a.size(0)), static_cast<int>(b.size(b_mn ? 1 : 0)),
        static_cast<int>(a.size(1)), status_dev_ptr(), num_sms(a), stream_of(a));
    TORCH_CHECK(err == nullptr, "gemm_scatter: ", err);
    g_launches += 1;
}

// out[i] = sum_w slices[w, i] in fp32; `slices` is [W, n] bf16, `out` is [n] bf16 or fp32.
void reduce_slices(const Tensor& slices, Tensor out) {
    TORCH_CHECK(slices.is_cuda() && is_bf16(slices) && slices.is_contiguous() && slices.dim() >= 2 && aligned16(slices),
                "reduce_slices: `slices` must be a contiguous bf16 CUDA tensor [W, ...]");
    const int64_t W = slices.size(0), n = slices.numel() / W;
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() == n && aligned16(out) && n % 8 == 0 &&
                    (is_bf16(out) || out.scalar_type() == at::kFloat) && W >= 1 && W <= 8,
                "reduce_slices: `out` must be a contiguous bf16/fp32 CUDA tensor of one slice (multiple of 8 elements)");
    c10::cuda::CUDAGuard guard(out.device());
    fs2::comm_reduce_slices(slices.data_ptr(), static_cast<int>(W), n, out.data_ptr(), out.scalar_type() == at::kFloat,
                            stream_of(out));
    g_launches += 1;
}

// out[M,N] = A * B^T with one operand assembled from the ranks' row shards inside the kernel. The shards sit at
// `shard_byte_off` of every arena, the local scratch for the assembled operand at `gathered_byte_off` of this
// rank's arena, the per-block flags at `flags_byte_off`.
void gemm_allgather(const std::vector<int64_t>& ptrs, int64_t rank, int64_t shard_byte_off, int64_t rows_per_rank,
                    const Tensor& other, int64_t gathered_byte_off, int64_t flags_byte_off, int64_t epoch,
                    bool gather_b, Tensor out, int64_t ncopy, bool other_mn) {
    TORCH_CHECK(!(other_mn && gather_b), "gemm_allgather: an MN-major local operand needs gather of A");
    TORCH_CHECK(other.is_cuda() && is_bf16(other) && other.dim() == 2 && other.is_contiguous() && aligned16(other),
                "gemm_allgather: the local operand must be a contiguous bf16 CUDA matrix");
    TORCH_CHECK(out.is_cuda() && is_bf16(out) && out.dim() == 2 && out.is_contiguous() && aligned16(out),
                "gemm_allgather: `out` must be a contiguous bf16 CUDA matrix");
    const int64_t world = static_cast<int64_t>(ptrs.size());
    TORCH_CHECK(world >= 1 && world <= 8 && rank >= 0 && rank < world, "gemm_allgather: bad world/rank");
    const int64_t K = other_mn ? other.size(0) : other.size(1);
    const int64_t M = gather_b ? other.size(0) : rows_per_rank * world;
    const int64_t N = gather_b ? rows_per_rank * world : (other_mn ? other.size(1) : other.size(0));
    TORCH_CHECK(out.size(0) == M && out.size(1) == N && K % 8 == 0 && N % 8 == 0, "gemm_allgather: shape mismatch");
    TORCH_CHECK(shard_byte_off % 16 == 0 && gathered_byte_off % 1024 == 0 && flags_byte_off % 4 == 0,
                "gemm_allgather: unaligned arena offsets");
    // a negative shard offset means: rank r keeps its shard at slice r of its own gathered buffer
    const bool inplace = shard_byte_off < 0;
    const void* shards[8];
    for (int64_t r = 0; r < world; ++r) {
        const int64_t off = inplace ? gathered_byte_off + r * rows_per_rank * K * 2 : shard_byte_off;
        shards[r] = reinterpret_cast<const void*>(ptrs[static_cast<size_t>(r)] + off);
    }
    const int64_t mine = ptrs[static_cast<size_t>(rank)];
    check_status();
    c10::cuda::CUDAGuard guard(other.device());
    TORCH_CHECK(cudaSetDevice(other.get_device()) == cudaSuccess, "gemm_allgather: cudaSetDevice failed");
    const char* err = fs2::gemm_allgather_bf16_tcgen05(
        shards, static_cast<int>(world), static_cast<int>(rank), static_cast<int>(rows_per_rank), other.data_ptr(),
        reinterpret_cast<void*>(mine + gathered_byte_off), reinterpret_cast<unsigned int*>(mine + flags_byte_off),
        static_cast<unsigned int>(epoch), gather_b, out.data_ptr(), static_cast<int>(M), static_cast<int>(N),
        static_cast<int>(K), static_cast<int>(ncopy), inplace, status_dev_ptr(), num_sms(other), stream_of(other),
        other_mn);
    TORCH_CHECK(err == nullptr, "gemm_allgather: ", err);
    g_launches += 1;
}

// ---------------------------------------------------------------------- norms
std::tuple<Tensor, Tensor> rms_norm_fwd(const Tensor& x, const Tensor& w, double eps) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && w.is_contiguous(), "rms_norm_fwd: bad input");
    TORCH_CHECK(x.scalar_type() == w.scalar_type() && (is_bf16(x) || x.scalar_type() == at::kFloat),
                "rms_norm_fwd: dtype must be bf16 or fp32 and match the weight");
    const int rows = static_cast<int>(x.size(0)), D = static_cast<int>(x.size(1));
    TORCH_CHECK(D % 8 == 0 && D <= 65536 && w.numel() == D && aligned16(x) && aligned16(w), "rms_norm_fwd: bad dim");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = at::empty_like(x);
    Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
    if (rows > 0)
        fs2::rms_norm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, D,
                          static_cast<float>(eps), is_bf16(x), num_sms(x), stream_of(x));
    g_launches += 1;
    return {y, rstd};
}

// h = x + res, y = rms_norm(h) * w in one pass; returns (h, y, rstd).
std::tuple<Tensor, Tensor, Tensor> add_rms_norm_fwd(const Tensor& x, const Tensor& res, const Tensor& w, double eps) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && w.is_contiguous() && res.is_contiguous() &&
                    res.sizes() == x.sizes() && res.device() == x.device(),
                "add_rms_norm_fwd: bad input");
    TORCH_CHECK(x.scalar_type() == w.scalar_type() && x.scalar_type() == res.scalar_type() &&
                    (is_bf16(x) || x.scalar_type() == at::kFloat),
                "add_rms_norm_fwd: dtype must be bf16 or fp32 and match the weight and the residual");
    const int rows = static_cast<int>(x.size(0)), D = static_cast<int>(x.size(1));
    TORCH_CHECK(D % 8 == 0 && D <= 65536 && w.numel() == D && aligned16(x) && aligned16(w) && aligned16(res),
                "add_rms_norm_fwd: bad dim");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor h = at::empty_like(x);
    Tensor y = at::empty_like(x);
    Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
    if (rows > 0)
        fs2::rms_norm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, D,
                          static_cast<float>(eps), is_bf16(x), num_sms(x), stream_of(x), res.data_ptr(),
                          h.data_ptr());
    g_launches += 1;
    return {h, y, rstd};
}

std::tuple<Tensor, Tensor> rms_norm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd,
                                        const std::optional<Tensor>& dres) {
    TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && x.is_contiguous() && dy.sizes() == x.sizes(),
                "rms_norm_bwd: bad input");
    TORCH_CHECK(dy.scalar_type() == x.scalar_type(), "rms_norm_bwd: dtype mismatch");
    const void* dres_ptr = nullptr;
    if (dres.has_value()) {
        TORCH_CHECK(dres->is_cuda() && dres->is_contiguous() && dres->sizes() == x.sizes() &&
                        dres->scalar_type() == x.scalar_type() && aligned16(*dres),
                    "rms_norm_bwd: the residual gradient must match x");
        dres_ptr = dres->data_ptr();
    }
    const int rows = static_cast<int>(x.size(0)), D = static_cast<int>(x.size(1));
    c10::cuda::CUDAGuard guard(x.device());
    Tensor dx = at::empty_like(x);
    Tensor dw = at::zeros({D}, x.options().dtype(at::kFloat));
    if (rows > 0) {
        const int grid = fs2::norm_bwd_grid(rows, num_sms(x));
        Tensor part = at::empty({grid, D}, x.options().dtype(at::kFloat));
        fs2::rms_norm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                          part.data_ptr<float>(), dw.data_ptr<float>(), rows, D, is_bf16(x), num_sms(x),
                          stream_of(x), dres_ptr);
        g_launches += 2;
    } else if (dres.has_value()) {
        dx.copy_(*dres);
    }
    return {dx, dw};
}

std::tuple<Tensor, Tensor, Tensor> layer_norm_fwd(const Tensor& x, const Tensor& w, const Tensor& b, double eps,
                                                  bool gelu) {
    TORCH_CHECK(!gelu || is_bf16(x), "layer_norm_fwd: the fused GELU needs bf16");
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && w.is_contiguous() && b.is_contiguous(),
                "layer_norm_fwd: bad input");
    TORCH_CHECK(x.scalar_type() == w.scalar_type() && x.scalar_type() == b.scalar_type() &&
                    (is_bf16(x) || x.scalar_type() == at::kFloat),
                "layer_norm_fwd: dtype must be bf16 or fp32 and match weight/bias");
    const int rows = static_cast<int>(x.size(0)), D = static_cast<int>(x.size(1));
    TORCH_CHECK(D % 8 == 0 && D <= 65536 && w.numel() == D && b.numel() == D && aligned16(x) && aligned16(w) &&
                    aligned16(b),
                "layer_norm_fwd: bad dim");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = at::empty_like(x);
    Tensor mean = at::empty({rows}, x.options().dtype(at::kFloat));
    Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
    if (rows > 0)
        fs2::layer_norm_fwd(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), mean.data_ptr<float>(),
                            rstd.data_ptr<float>(), rows, D, static_cast<float>(eps), is_bf16(x), num_sms(x),
                            stream_of(x), gelu);
    g_launches += 1;
    return {y, mean, rstd};
}

std::tuple<Tensor, Tensor, Tensor> layer_norm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w,
                                                  const Tensor& mean, const Tensor& rstd,
                                                  const std::optional<Tensor>& b_for_gelu) {
    TORCH_CHECK(!b_for_gelu.has_value() || (is_bf16(x) && is_bf16(*b_for_gelu) && b_for_gelu->is_contiguous() &&
                                            b_for_gelu->numel() == x.size(1)),
                "layer_norm_bwd: the fused GELU needs bf16 and the bias");
    TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && x.is_contiguous() && dy.sizes() == x.sizes(),
                "layer_norm_bwd: bad input");
    const int rows = static_cast<int>(x.size(0)), D = static_cast<int>(x.size(1));
    c10::cuda::CUDAGuard guard(x.device());
    Tensor dx = at::empty_like(x);
    Tensor dw = at::zeros({D}, x.options().dtype(at::kFloat));
    Tensor db = at::zeros({D}, x.options().dtype(at::kFloat));
    if (rows > 0) {
        const int grid = fs2::norm_bwd_grid(rows, num_sms(x));
        Tensor part = at::empty({2, grid, D}, x.options().dtype(at::kFloat));
        fs2::layer_norm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr<float>(),
                            rstd.data_ptr<float>(), dx.data_ptr(), part[0].data_ptr<float>(),
                            part[1].data_ptr<float>(), dw.data_ptr<float>(), db.data_ptr<float>(), rows, D,
                            is_bf16(x), num_sms(x), stream_of(x),
                            b_for_gelu.has_value() ? b_for_gelu->data_ptr() : nullptr);
        g_launches += 3;
    }
    return {dx, dw, db};
}

// ------------------------------------------------------- vocabulary-parallel embedding
Tensor embed_vocab_parallel_fwd(const Tensor& ids, const Tensor& table, int64_t lo, double scale) {
    TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && table.is_cuda() &&
                    is_bf16(table) && table.dim() == 2 && table.is_contiguous() && table.size(1) % 8 == 0 &&
                    aligned16(table),
                "embed_vocab_parallel_fwd: ids must be int64, the table shard a contiguous bf16 [rows, D] with D % 8 == 0");
    c10::cuda::CUDAGuard guard(table.device());
    auto shape = ids.sizes().vec();
    shape.push_back(table.size(1));
    Tensor out = at::empty(shape, table.options());
    fs2::embed_vocab_parallel_fwd(ids.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()) : nullptr,
                                  table.data_ptr(), out.data_ptr(), static_cast<size_t>(ids.numel()),
                                  static_cast<int>(table.size(1)), lo, table.size(0), static_cast<float>(scale),
                                  stream_of(table));
    g_launches += 1;
    return out;
}

Tensor embed_vocab_parallel_bwd(const Tensor& ids, const Tensor& dout, int64_t rows, int64_t lo, double scale) {
    TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && dout.is_cuda() &&
                    is_bf16(dout) && dout.is_contiguous() && dout.size(-1) % 8 == 0 && aligned16(dout) &&
                    dout.numel() == ids.numel() * dout.size(-1),
                "embed_vocab_parallel_bwd: bad tensors");
    c10::cuda::CUDAGuard guard(dout.device());
    Tensor dtable = at::zeros({rows, dout.size(-1)}, dout.options().dtype(at::kFloat));
    fs2::embed_vocab_parallel_bwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), dout.data_ptr(),
                                  dtable.data_ptr<float>(), static_cast<size_t>(ids.numel()),
                                  static_cast<int>(dout.size(-1)), lo, rows, static_cast<float>(scale), stream_of(dout));
    g_launches += 1;
    return dtable;
}

// --------------------------------------------------------------------- SwiGLU
Tensor swiglu_fwd(const Tensor& gu) {
    TORCH_CHECK(gu.is_cuda() && is_bf16(gu) && gu.dim() == 2 && gu.is_contiguous() && gu.size(1) % 16 == 0 &&
                    aligned16(gu),
                "swiglu_fwd: expects contiguous bf16 [rows, 2F] with F % 8 == 0");
    const int64_t rows = gu.size(0), F = gu.size(1) / 2;
    c10::cuda::CUDAGuard guard(gu.device());
    Tensor y = at::empty({rows, F}, gu.options());
    if (rows > 0)
        fs2::swiglu_fwd(gu.data_ptr(), y.data_ptr(), static_cast<size_t>(rows), static_cast<int>(F), num_sms(gu),
                        stream_of(gu));
    g_launches += 1;
    return y;
}

// SwiGLU of separate gate / up matrices, bounded by a device-resident tile count (rows beyond stay untouched).
namespace {
const int* tiles_ptr(const std::optional<Tensor>& num_tiles, const Tensor& like) {
    if (!num_tiles.has_value()) return nullptr;
    TORCH_CHECK(num_tiles->is_cuda() && num_tiles->scalar_type() == at::kInt && num_tiles->numel() >= 1 &&
                    num_tiles->device() == like.device(),
                "`num_tiles` must be an int32 CUDA tensor on the same device");
    return num_tiles->data_ptr<int>();
}
}  // namespace

Tensor swiglu2_fwd(const Tensor& g, const Tensor& u, const std::optional<Tensor>& num_tiles) {
    TORCH_CHECK(g.is_cuda() && is_bf16(g) && is_bf16(u) && g.dim() == 2 && g.is_contiguous() && u.is_contiguous() &&
                    g.sizes() == u.sizes() && g.size(1) % 8 == 0 && aligned16(g) && aligned16(u),
                "swiglu2_fwd: expects two contiguous bf16 [rows, F] matrices with F % 8 == 0");
    c10::cuda::CUDAGuard guard(g.device());
    Tensor y = at::empty_like(g);
    fs2::swiglu2_fwd(g.data_ptr(), u.data_ptr(), y.data_ptr(), static_cast<size_t>(g.size(0)),
                     static_cast<int>(g.size(1)), tiles_ptr(num_tiles, g), num_sms(g), stream_of(g));
    g_launches += 1;
    return y;
}

std::tuple<Tensor, Tensor> swiglu2_bwd(const Tensor& dy, const Tensor& g, const Tensor& u,
                                       const std::optional<Tensor>& num_tiles) {
    TORCH_CHECK(dy.is_cuda() && is_bf16(dy) && dy.is_contiguous() && g.is_contiguous() && u.is_contiguous() &&
                    dy.sizes() == g.sizes() && g.sizes() == u.sizes() && aligned16(dy),
                "swiglu2_bwd: bad input");
    c10::cuda::CUDAGuard guard(g.device());
    Tensor dg = at::empty_like(g), du = at::empty_like(u);
    fs2::swiglu2_bwd(dy.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(), du.data_ptr(),
                     static_cast<size_t>(g.size(0)), static_cast<int>(g.size(1)), tiles_ptr(num_tiles, g), num_sms(g),
                     stream_of(g));
    g_launches += 1;
    return {dg, du};
}

void copy_rows_bounded(Tensor dst, const Tensor& src, const std::optional<Tensor>& num_tiles) {
    TORCH_CHECK(dst.is_cuda() && src.is_cuda() && dst.dim() == 2 && dst.is_contiguous() && src.is_contiguous() &&
                    dst.sizes() == src.sizes() && dst.scalar_type() == src.scalar_type() &&
                    (dst.size(1) * dst.element_size()) % 16 == 0 && aligned16(dst) && aligned16(src),
                "copy_rows_bounded: two contiguous [rows, D] matrices of the same type with 16-byte rows");
    c10::cuda::CUDAGuard guard(dst.device());
    fs2::copy_rows_bounded(dst.data_ptr(), src.data_ptr(), static_cast<size_t>(dst.size(0)),
                           static_cast<size_t>(dst.size(1) * dst.element_size()), tiles_ptr(num_tiles, dst),
                           num_sms(dst), stream_of(dst));
    g_launches += 1;
}

Tensor swiglu_bwd(const Tensor& dy, const Tensor& gu) {
    TORCH_CHECK(dy.is_cuda() && is_bf16(dy) && dy.is_contiguous() && gu.is_contiguous() && dy.dim() == 2 &&
                    gu.size(0) == dy.size(0) && gu.size(1) == 2 * dy.size(1),
                "swiglu_bwd: bad input");
    c10::cuda::CUDAGuard guard(gu.device());
    Tensor dgu = at::empty_like(gu);
    if (gu.size(0) > 0)
        fs2::swiglu_bwd(dy.data_ptr(), gu.data_ptr(), dgu.data_ptr(), static_cast<size_t>(gu.size(0)),
                        static_cast<int>(dy.size(1)), num_sms(gu), stream_of(gu));
    g_launches += 1;
    return dgu;
}

// ----------------------------------------------------------------------- RoPE
void rope_inplace(Tensor x, const Tensor& freqs, const Tensor& pos, bool inverse) {
    TORCH_CHECK(x.is_cuda() && is_bf16(x) && x.dim() == 3 && x.stride(2) == 1, "rope_inplace: x must be bf16 [T, heads, D]");
    TORCH_CHECK(freqs.is_cuda() && freqs.scalar_type() == at::kFloat && freqs.is_contiguous() && freqs.dim() == 3 &&
                    freqs.size(1) * 2 == x.size(2) && freqs.size(2) == 2,
                "rope_inplace: freqs must be fp32 [L, D/2, 2]");
    TORCH_CHECK(pos.is_cuda() && pos.scalar_type() == at::kInt && pos.is_contiguous() && pos.numel() == x.size(0),
                "rope_inplace: positions must be int32 [T]");
    const int D = static_cast<int>(x.size(2));
    TORCH_CHECK(D % 8 == 0 && x.stride(0) % 8 == 0 && x.stride(1) % 8 == 0 && aligned16(x), "rope_inplace: alignment");
    c10::cuda::CUDAGuard guard(x.device());
    fs2::rope_inplace(x.data_ptr(), freqs.data_ptr<float>(), pos.data_ptr<int>(), static_cast<size_t>(x.size(0)),
                      static_cast<int>(x.size(1)), D, static_cast<size_t>(x.stride(0)),
                      static_cast<size_t>(x.stride(1)), static_cast<int>(freqs.size(0)), inverse, num_sms(x),
                      stream_of(x));
    g_launches += 1;
}

// ------------------------------------------------------------------------ MoE
// logits [T, E] -> (expert_ids [T, k] int32, gates [T, k] fp32, counts [E] int32, prob_sum [E] fp32 or empty)
std::tuple<Tensor, Tensor, Tensor, Tensor> moe_route(const Tensor& logits, int64_t k, bool softmax_gate,
                                                     bool with_prob_sum) {
    TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous() &&
                    (is_bf16(logits) || logits.scalar_type() == at::kFloat),
                "moe_route: logits must be a contiguous bf16/fp32 [T, E] CUDA tensor");
    const int64_t T = logits.size(0), E = logits.size(1);
    TORCH_CHECK(E >= 1 && E <= 256 && k >= 1 && k <= 8 && k <= E, "moe_route: up to 256 experts and top-8 are supported");
    c10::cuda::CUDAGuard guard(logits.device());
    auto iopt = logits.options().dtype(at::kInt);
    auto fopt = logits.options().dtype(at::kFloat);
    Tensor ids = at::empty({T, k}, iopt), gates = at::empty({T, k}, fopt), counts = at::zeros({E}, iopt);
    Tensor prob_sum = with_prob_sum ? at::zeros({E}, fopt) : at::empty({0}, fopt);
    fs2::moe_route(logits.data_ptr(), is_bf16(logits), static_cast<int>(T), static_cast<int>(E), static_cast<int>(k),
                   softmax_gate, ids.data_ptr<int>(), gates.data_ptr<float>(), counts.data_ptr<int>(),
                   with_prob_sum ? prob_sum.data_ptr<float>() : nullptr, stream_of(logits));
    g_launches += 1;
    return {ids, gates, counts, prob_sum};
}

// x [T, D] bf16 -> (routed [T*k, D] bf16 in expert order, src_row [T*k] int32, inv [T, k] int32, offsets [E+1] int32)
std::tuple<Tensor, Tensor, Tensor, Tensor> moe_dispatch(const Tensor& x, const Tensor& expert_ids, const Tensor& gates,
                                                        const Tensor& counts, bool scale_by_gate) {
    TORCH_CHECK(x.is_cuda() && is_bf16(x) && x.dim() == 2 && x.is_contiguous() && x.size(1) % 8 == 0 && aligned16(x),
                "moe_dispatch: x must be a contiguous bf16 [T, D] CUDA tensor with D % 8 == 0");
    TORCH_CHECK(expert_ids.scalar_type() == at::kInt && expert_ids.is_contiguous() && expert_ids.dim() == 2 &&
                    expert_ids.size(0) == x.size(0) && gates.scalar_type() == at::kFloat && gates.is_contiguous() &&
                    gates.sizes() == expert_ids.sizes() && counts.scalar_type() == at::kInt && counts.is_contiguous(),
                "moe_dispatch: bad routing tensors");
    const int64_t T = x.size(0), D = x.size(1), k = expert_ids.size(1), E = counts.numel();
    c10::cuda::CUDAGuard guard(x.device());
    auto iopt = x.options().dtype(at::kInt);
    Tensor offsets = at::empty({E + 1}, iopt), cursor = at::empty({E}, iopt);
    Tensor routed = at::empty({T * k, D}, x.options()), src_row = at::empty({T * k}, iopt), inv = at::empty({T, k}, iopt);
    fs2::moe_offsets(counts.data_ptr<int>(), offsets.data_ptr<int>(), cursor.data_ptr<int>(), static_cast<int>(E),
                     stream_of(x));
    fs2::moe_dispatch(x.data_ptr(), expert_ids.data_ptr<int>(), gates.data_ptr<float>(), offsets.data_ptr<int>(),
                      cursor.data_ptr<int>(), routed.data_ptr(), src_row.data_ptr<int>(), inv.data_ptr<int>(),
                      static_cast<int>(T), static_cast<int>(k), static_cast<int>(D), scale_by_gate, stream_of(x));
    g_launches += 2;
    return {routed, src_row, inv, offsets};
}

// ------------------------------------------------------------------ wav2vec 2.0 objective
// returns (logits [P, K + 1] fp32, lse [P] fp32, loss_sum [1] fp32)
std::tuple<Tensor, Tensor, Tensor> w2v_contrastive_fwd(const Tensor& x, const Tensor& tgt, const Tensor& distractors,
                                                       double temp) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && tgt.is_contiguous() && tgt.sizes() == x.sizes() &&
                    x.scalar_type() == tgt.scalar_type() && (is_bf16(x) || x.scalar_type() == at::kFloat),
                "w2v_contrastive_fwd: x and targets must be contiguous [P, M] bf16/fp32 CUDA tensors");
    TORCH_CHECK(distractors.scalar_type() == at::kInt && distractors.is_contiguous() && distractors.dim() == 2 &&
                    distractors.size(0) == x.size(0) && x.size(1) <= 1024,
                "w2v_contrastive_fwd: distractors must be int32 [P, K]; feature dim <= 1024");
    const int64_t P = x.size(0), M = x.size(1), K = distractors.size(1);
    c10::cuda::CUDAGuard guard(x.device());
    auto fopt = x.options().dtype(at::kFloat);
    Tensor logits = at::empty({P, K + 1}, fopt), lse = at::empty({P}, fopt), loss = at::zeros({1}, fopt);
    fs2::w2v_contrastive_fwd(x.data_ptr(), tgt.data_ptr(), is_bf16(x), distractors.data_ptr<int>(), static_cast<int>(P),
                             static_cast<int>(K), static_cast<int>(M), static_cast<float>(temp),
                             logits.data_ptr<float>(), lse.data_ptr<float>(), loss.data_ptr<float>(), stream_of(x));
    g_launches += 1;
    return {logits, lse, loss};
}

// returns (dx [P, M] fp32, dtgt [P, M] fp32)
std::tuple<Tensor, Tensor> w2v_contrastive_bwd(const Tensor& x, const Tensor& tgt, const Tensor& distractors,
                                               const Tensor& logits, const Tensor& lse, const Tensor& scale,
                                               double temp) {
    const int64_t P = x.size(0), M = x.size(1), K = distractors.size(1);
    TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::kFloat && scale.numel() == 1 && logits.is_contiguous() &&
                    lse.is_contiguous() && logits.numel() == P * (K + 1) && lse.numel() == P,
                "w2v_contrastive_bwd: bad saved tensors");
    c10::cuda::CUDAGuard guard(x.device());
    auto fopt = x.options().dtype(at::kFloat);
    Tensor dx = at::empty({P, M}, fopt), dtgt = at::zeros({P, M}, fopt);
    fs2::w2v_contrastive_bwd(x.data_ptr(), tgt.data_ptr(), is_bf16(x), distractors.data_ptr<int>(),
                             logits.data_ptr<float>(), lse.data_ptr<float>(), scale.data_ptr<float>(),
                             static_cast<int>(P), static_cast<int>(K), static_cast<int>(M), static_cast<float>(temp),
                             dx.data_ptr<float>(), dtgt.data_ptr<float>(), stream_of(x));
    g_launches += 1;
    return {dx, dtgt};
}

// First wav2vec 2.0 feature-extractor layer: conv (1 input channel, kernel width 10) + bias [+ LayerNorm + GELU],
// channels-last output [B, t_pad, C] with rows >= t_valid zeroed.
bool w2v_first_conv_supported(int64_t C, int64_t kernel_width) {
    return fs2::w2v_first_conv_supported(static_cast<int>(C), static_cast<int>(kernel_width));
}

namespace {
const void* opt_ptr(const std::optional<Tensor>& t, int64_t C, const Tensor& like, const char* what) {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->is_cuda() && is_bf16(*t) && t->is_contiguous() && t->numel() == C && t->device() == like.device(),
                "w2v_first_conv: `", what, "` must be a contiguous bf16 CUDA tensor of C elements");
    return t->data_ptr();
}
}  // namespace

Tensor w2v_first_conv_fwd(const Tensor& x, const Tensor& w, const std::optional<Tensor>& bias,
                          const std::optional<Tensor>& lnw, const std::optional<Tensor>& lnb, int64_t stride,
                          int64_t t_pad, double eps) {
    TORCH_CHECK(x.is_cuda() && is_bf16(x) && x.dim() == 2 && x.is_contiguous() && w.is_cuda() && is_bf16(w) &&
                    w.is_contiguous() && w.dim() == 2,
                "w2v_first_conv_fwd: x must be a contiguous bf16 [B, L] waveform, w a contiguous bf16 [C, 10]");
    const int64_t B = x.size(0), L = x.size(1), C = w.size(0), KW = w.size(1);
    TORCH_CHECK(fs2::w2v_first_conv_supported(static_cast<int>(C), static_cast<int>(KW)) && stride >= 1 && L >= KW,
                "w2v_first_conv_fwd: unsupported shape");
    TORCH_CHECK(lnw.has_value() == lnb.has_value(), "w2v_first_conv_fwd: LayerNorm weight and bias come together");
    const int64_t t_valid = (L - KW) / stride + 1;
    TORCH_CHECK(t_pad >= t_valid, "w2v_first_conv_fwd: `t_pad` is smaller than the number of output positions");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = at::empty({B, t_pad, C}, x.options());
    fs2::w2v_first_conv_fwd(x.data_ptr(), w.data_ptr(), opt_ptr(bias, C, x, "bias"), opt_ptr(lnw, C, x, "ln weight"),
                            opt_ptr(lnb, C, x, "ln bias"), y.data_ptr(), static_cast<int>(B), static_cast<int>(L),
                            static_cast<int>(t_valid), static_cast<int>(t_pad), static_cast<int>(C),
                            static_cast<int>(stride), static_cast<float>(eps), num_sms(x), stream_of(x));
    g_launches += 1;
    return y;
}

// returns fp32 (dw [C, 10], dbias [C], dlnw [C], dlnb [C]); entries for absent inputs are empty tensors
std::tuple<Tensor, Tensor, Tensor, Tensor> w2v_first_conv_bwd(const Tensor& dy, const Tensor& x, const Tensor& w,
                                                              const std::optional<Tensor>& bias,
                                                              const std::optional<Tensor>& lnw,
                                                              const std::optional<Tensor>& lnb, int64_t stride,
                                                              double eps) {
    TORCH_CHECK(dy.is_cuda() && is_bf16(dy) && dy.dim() == 3 && dy.is_contiguous() && x.is_contiguous() &&
                    dy.size(0) == x.size(0) && dy.size(2) == w.size(0),
                "w2v_first_conv_bwd: dy must be a contiguous bf16 [B, t_pad, C] tensor");
    const int64_t B = x.size(0), L = x.size(1), C = w.size(0), KW = w.size(1), t_pad = dy.size(1);
    const int64_t t_valid = (L - KW) / stride + 1;
    TORCH_CHECK(t_pad >= t_valid, "w2v_first_conv_bwd: dy has fewer rows than output positions");
    c10::cuda::CUDAGuard guard(x.device());
    auto fopt = x.options().dtype(at::kFloat);
    Tensor dw = at::zeros({C, KW}, fopt);
    Tensor db = bias.has_value() ? at::zeros({C}, fopt) : at::empty({0}, fopt);
    Tensor dlw = lnw.has_value() ? at::zeros({C}, fopt) : at::empty({0}, fopt);
    Tensor dlb = lnb.has_value() ? at::zeros({C}, fopt) : at::empty({0}, fopt);
    fs2::w2v_first_conv_bwd(x.data_ptr(), w.data_ptr(), opt_ptr(bias, C, x, "bias"), opt_ptr(lnw, C, x, "ln weight"),
                            opt_ptr(lnb, C, x, "ln bias"), dy.data_ptr(), dw.data_ptr<float>(),
                            bias.has_value() ? db.data_ptr<float>() : nullptr,
                            lnw.has_value() ? dlw.data_ptr<float>() : nullptr,
                            lnb.has_value() ? dlb.data_ptr<float>() : nullptr, static_cast<int>(B), static_cast<int>(L),
                            static_cast<int>(t_valid), static_cast<int>(t_pad), static_cast<int>(C),
                            static_cast<int>(stride), static_cast<float>(eps), num_sms(x), stream_of(x));
    g_launches += 1;
    return {dw, db, dlw, dlb};
}

// returns (q [R, E], hard_idx [R], sel [R], prob_sum [G, V], hard_count [G, V], y_soft [R, V] or empty)
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor> w2v_quantize_fwd(const Tensor& logits,
                                                                            const std::optional<Tensor>& noise,
                                                                            const Tensor& entries, int64_t G, double tau,
                                                                            bool training, bool keep_soft) {
    TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous() && entries.is_contiguous() &&
                    entries.dim() == 2 && logits.scalar_type() == entries.scalar_type() &&
                    (is_bf16(logits) || logits.scalar_type() == at::kFloat),
                "w2v_quantize_fwd: logits [R, V] and entries [G * V, E] must be contiguous bf16/fp32 CUDA tensors");
    const int64_t R = logits.size(0), V = logits.size(1), E = entries.size(1);
    TORCH_CHECK(G >= 1 && R % G == 0 && entries.size(0) == G * V && V <= 512, "w2v_quantize_fwd: bad shapes");
    const float* np = nullptr;
    if (noise.has_value()) {
        TORCH_CHECK(noise->scalar_type() == at::kFloat && noise->is_contiguous() && noise->sizes() == logits.sizes(),
                    "w2v_quantize_fwd: noise must be fp32 [R, V]");
        np = noise->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(logits.device());
    auto fopt = logits.options().dtype(at::kFloat);
    auto iopt = logits.options().dtype(at::kInt);
    Tensor q = at::empty({R, E}, logits.options()), hard_idx = at::empty({R}, iopt), sel = at::empty({R}, iopt);
    Tensor prob_sum = at::zeros({G, V}, fopt), hard_count = at::zeros({G, V}, fopt);
    Tensor y_soft = (training && keep_soft) ? at::empty({R, V}, fopt) : at::empty({0}, fopt);
    fs2::w2v_quantize_fwd(logits.data_ptr(), np, entries.data_ptr(), is_bf16(logits), static_cast<int>(R),
                          static_cast<int>(G), static_cast<int>(V), static_cast<int>(E), static_cast<float>(tau), training,
                          hard_idx.data_ptr<int>(), sel.data_ptr<int>(), prob_sum.data_ptr<float>(),
                          hard_count.data_ptr<float>(), y_soft.numel() ? y_soft.data_ptr<float>() : nullptr, q.data_ptr(),
                          stream_of(logits));
    g_launches += 1;
    return {q, hard_idx, sel, prob_sum, hard_count, y_soft};
}

// returns (dlogits [R, V] fp32, dentries [G * V, E] fp32)
std::tuple<Tensor, Tensor> w2v_quantize_bwd(const Tensor& dq, const Tensor& entries, const Tensor& y_soft,
                                            const Tensor& sel, int64_t G, double tau) {
    TORCH_CHECK(dq.is_cuda() && dq.is_contiguous() && dq.dim() == 2 && entries.is_contiguous() &&
                    dq.scalar_type() == entries.scalar_type() && y_soft.scalar_type() == at::kFloat &&
                    y_soft.is_contiguous() && sel.scalar_type() == at::kInt,
                "w2v_quantize_bwd: bad tensors");
    const int64_t R = dq.size(0), E = dq.size(1), V = y_soft.size(1);
    TORCH_CHECK(entries.size(0) == G * V && entries.size(1) == E && y_soft.size(0) == R && sel.numel() == R,
                "w2v_quantize_bwd: bad shapes");
    c10::cuda::CUDAGuard guard(dq.device());
    auto fopt = dq.options().dtype(at::kFloat);
    Tensor dlogits = at::empty({R, V}, fopt), dentries = at::zeros({G * V, E}, fopt);
    fs2::w2v_quantize_bwd(dq.data_ptr(), entries.data_ptr(), is_bf16(dq), y_soft.data_ptr<float>(), sel.data_ptr<int>(),
                          static_cast<int>(R), static_cast<int>(G), static_cast<int>(V), static_cast<int>(E),
                          static_cast<float>(tau), dlogits.data_ptr<float>(), dentries.data_ptr<float>(), stream_of(dq));
    g_launches += 1;
    return {dlogits, dentries};
}

fs2::CommPeers make_peers(const std::vector<int64_t>& ptrs, int64_t rank, double wait_limit_s);

// Expert-parallel routing over the symmetric arena; see moe.h for the protocol.
std::tuple<Tensor, Tensor, Tensor, Tensor> moe_ep_layout(const std::vector<int64_t>& ptrs, int64_t rank,
                                                         const Tensor& counts, int64_t table_byte_off, int64_t slot,
                                                         int64_t epoch, double wait_limit_s) {
    const int64_t W = static_cast<int64_t>(ptrs.size()), E = counts.numel();
    TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kInt && counts.is_contiguous() && E % W == 0 && E <= 256,
                "moe_ep_layout: counts must be an int32 CUDA vector whose length is a multiple of the world size");
    TORCH_CHECK(table_byte_off % 16 == 0, "moe_ep_layout: unaligned table offset");
    c10::cuda::CUDAGuard guard(counts.device());
    auto iopt = counts.options();
    Tensor send_base = at::empty({E}, iopt), cursor = at::empty({E}, iopt), group_sizes = at::empty({E / W}, iopt),
           total = at::empty({1}, iopt);
    fs2::moe_ep_layout(make_peers(ptrs, rank, wait_limit_s), counts.data_ptr<int>(), table_byte_off, static_cast<int>(E),
                       send_base.data_ptr<int>(), cursor.data_ptr<int>(), group_sizes.data_ptr<int>(),
                       total.data_ptr<int>(), static_cast<int>(slot), static_cast<uint32_t>(epoch), status_dev_ptr(),
                       stream_of(counts));
    g_launches += 1;
    return {send_base, cursor, group_sizes, total};
}

// returns (send_base [E], limit [E], cursor [E], offsets [El + 1], group_sizes [El], tile_row0 [cap / 128],
//          tile_expert [cap / 128], num_tiles [1], total [1])
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor> moe_ep_layout_padded(
    const std::vector<int64_t>& ptrs, int64_t rank, const Tensor& counts, int64_t table_byte_off, int64_t inbox_byte_off,
    int64_t cap, int64_t D, int64_t slot, int64_t epoch, double wait_limit_s) {
    const int64_t W = static_cast<int64_t>(ptrs.size()), E = counts.numel();
    TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kInt && counts.is_contiguous() && E % W == 0 && E <= 256,
                "moe_ep_layout_padded: counts must be an int32 CUDA vector whose length is a multiple of the world size");
    const int64_t El = E / W;
    TORCH_CHECK(table_byte_off % 16 == 0 && inbox_byte_off % 16 == 0 && cap % 128 == 0 && cap >= 128 * El && D % 8 == 0,
                "moe_ep_layout_padded: the inbox must hold a multiple of 128 rows and at least 128 per local expert");
    c10::cuda::CUDAGuard guard(counts.device());
    auto iopt = counts.options();
    Tensor send_base = at::empty({E}, iopt), limit = at::empty({E}, iopt), cursor = at::empty({E}, iopt);
    Tensor offsets = at::empty({El + 1}, iopt), group_sizes = at::empty({El}, iopt);
    Tensor tile_row0 = at::empty({cap / 128}, iopt), tile_expert = at::empty({cap / 128}, iopt);
    Tensor num_tiles = at::empty({1}, iopt), total = at::empty({1}, iopt);
    void* inbox = reinterpret_cast<char*>(ptrs[static_cast<size_t>(rank)]) + inbox_byte_off;
    fs2::moe_ep_layout_padded(make_peers(ptrs, rank, wait_limit_s), counts.data_ptr<int>(), table_byte_off,
                              static_cast<int>(E), static_cast<int>(cap), send_base.data_ptr<int>(),
                              limit.data_ptr<int>(), cursor.data_ptr<int>(), offsets.data_ptr<int>(),
                              group_sizes.data_ptr<int>(), tile_row0.data_ptr<int>(), tile_expert.data_ptr<int>(),
                              num_tiles.data_ptr<int>(), total.data_ptr<int>(), inbox, static_cast<int>(D),
                              static_cast<int>(slot), static_cast<uint32_t>(epoch), status_dev_ptr(),
                              stream_of(counts));
    g_launches += 2;
    return {send_base, limit, cursor, offsets, group_sizes, tile_row0, tile_expert, num_tiles, total};
}

void moe_ep_push(const std::vector<int64_t>& ptrs, int64_t rank, const Tensor& x, const std::optional<Tensor>& expert_ids,
                 const std::optional<Tensor>& gates, const std::optional<Tensor>& send_base,
                 const std::optional<Tensor>& cursor, int64_t inbox_byte_off, Tensor dest, int64_t E, int64_t cap,
                 const std::optional<Tensor>& limit, const std::optional<Tensor>& dropped) {
    const int* limit_ptr = nullptr;
    int* dropped_ptr = nullptr;
    if (limit.has_value()) {
        TORCH_CHECK(limit->is_cuda() && limit->scalar_type() == at::kInt && limit->is_contiguous() && limit->numel() == E,
                    "moe_ep_push: limit must be int32 [E]");
        limit_ptr = limit->data_ptr<int>();
    }
    if (dropped.has_value()) {
        TORCH_CHECK(dropped->is_cuda() && dropped->scalar_type() == at::kInt && dropped->numel() == 1,
                    "moe_ep_push: dropped must be an int32 device scalar");
        dropped_ptr = dropped->data_ptr<int>();
    }
    TORCH_CHECK(x.is_cuda() && is_bf16(x) && x.dim() == 2 && x.is_contiguous() && x.size(1) % 8 == 0 && aligned16(x),
                "moe_ep_push: x must be a contiguous bf16 [T, D] CUDA tensor with D % 8 == 0");
    TORCH_CHECK(dest.scalar_type() == at::kInt && dest.is_contiguous() && dest.dim() == 2 && dest.size(0) == x.size(0),
                "moe_ep_push: dest must be int32 [T, k]");
    const bool assign = expert_ids.has_value();
    if (assign) {
        TORCH_CHECK(send_base.has_value() && cursor.has_value() && expert_ids->scalar_type() == at::kInt &&
                        expert_ids->is_contiguous() && expert_ids->sizes() == dest.sizes() &&
                        send_base->numel() == E && cursor->numel() == E,
                    "moe_ep_push: bad routing tensors");
    }
    const float* gp = nullptr;
    if (gates.has_value()) {
        TORCH_CHECK(gates->scalar_type() == at::kFloat && gates->is_contiguous() && gates->sizes() == dest.sizes(),
                    "moe_ep_push: gates must be fp32 [T, k]");
        gp = gates->data_ptr<float>();
    }
    TORCH_CHECK(inbox_byte_off % 16 == 0 && cap > 0 && E % static_cast<int64_t>(ptrs.size()) == 0, "moe_ep_push: bad arguments");
    c10::cuda::CUDAGuard guard(x.device());
    fs2::moe_ep_push(make_peers(ptrs, rank, 1.0), x.data_ptr(), assign ? expert_ids->data_ptr<int>() : nullptr, gp,
                     assign ? send_base->data_ptr<int>() : nullptr, assign ? cursor->data_ptr<int>() : nullptr,
                     inbox_byte_off, dest.data_ptr<int>(), static_cast<int>(x.size(0)), static_cast<int>(dest.size(1)),
                     static_cast<int>(x.size(1)), static_cast<int>(E), static_cast<int>(cap), assign, limit_ptr,
                     dropped_ptr, stream_of(x));
    g_launches += 1;
}

void moe_ep_pull(const std::vector<int64_t>& ptrs, int64_t rank, int64_t outbox_byte_off, const Tensor& dest,
                 const std::optional<Tensor>& gates, Tensor y, const std::optional<Tensor>& x,
                 const std::optional<Tensor>& dgate, int64_t cap, bool accumulate) {
    TORCH_CHECK(y.is_cuda() && is_bf16(y) && y.dim() == 2 && y.is_contiguous() && y.size(1) % 8 == 0 && aligned16(y),
                "moe_ep_pull: y must be a contiguous bf16 [T, D] CUDA tensor with D % 8 == 0");
    TORCH_CHECK(dest.scalar_type() == at::kInt && dest.is_contiguous() && dest.dim() == 2 && dest.size(0) == y.size(0) &&
                    dest.size(1) <= 8,
                "moe_ep_pull: dest must be int32 [T, k <= 8]");
    const float* gp = nullptr;
    if (gates.has_value()) {
        TORCH_CHECK(gates->scalar_type() == at::kFloat && gates->is_contiguous() && gates->sizes() == dest.sizes(),
                    "moe_ep_pull: gates must be fp32 [T, k]");
        gp = gates->data_ptr<float>();
    }
    const void* xp = nullptr;
    float* dgp = nullptr;
    if (x.has_value()) {
        TORCH_CHECK(dgate.has_value() && is_bf16(*x) && x->is_contiguous() && x->sizes() == y.sizes() &&
                        dgate->scalar_type() == at::kFloat && dgate->is_contiguous() && dgate->sizes() == dest.sizes(),
                    "moe_ep_pull: x must match y and dgate must be fp32 [T, k]");
        xp = x->data_ptr();
        dgp = dgate->data_ptr<float>();
    }
    TORCH_CHECK(outbox_byte_off % 16 == 0 && cap > 0, "moe_ep_pull: bad arguments");
    c10::cuda::CUDAGuard guard(y.device());
    fs2::moe_ep_pull(make_peers(ptrs, rank, 1.0), outbox_byte_off, dest.data_ptr<int>(), gp, y.data_ptr(), xp, dgp,
                     static_cast<int>(y.size(0)), static_cast<int>(dest.size(1)), static_cast<int>(y.size(1)),
                     static_cast<int>(cap), accumulate, stream_of(y));
    g_launches += 1;
}

// Dispatch into the 128-row padded, expert-sorted layout of the single-launch grouped GEMM. Nothing is read back
// to the host: the buffer is sized for the worst case (T * k + 128 * E rows) and the tile tables stay on the device.
// returns (routed [cap, D] (padding rows zero), src_row [cap] (-1 on padding rows), inv [T, k], offsets [E + 1],
//          tile_row0 [cap / 128], tile_expert [cap / 128], num_tiles [1])
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor> moe_dispatch_padded(const Tensor& x,
                                                                                   const Tensor& expert_ids,
                                                                                   const Tensor& gates,
                                                                                   const Tensor& counts,
                                                                                   bool scale_by_gate) {
    TORCH_CHECK(x.is_cuda() && is_bf16(x) && x.dim() == 2 && x.is_contiguous() && x.size(1) % 8 == 0 && aligned16(x),
                "moe_dispatch_padded: x must be a contiguous bf16 [T, D] CUDA tensor with D % 8 == 0");
    TORCH_CHECK(expert_ids.scalar_type() == at::kInt && expert_ids.is_contiguous() && expert_ids.dim() == 2 &&
                    expert_ids.size(0) == x.size(0) && gates.scalar_type() == at::kFloat && gates.is_contiguous() &&
                    gates.sizes() == expert_ids.sizes() && counts.scalar_type() == at::kInt && counts.is_contiguous(),
                "moe_dispatch_padded: bad routing tensors");
    const int64_t T = x.size(0), D = x.size(1), k = expert_ids.size(1), E = counts.numel();
    TORCH_CHECK(E >= 1 && E <= 256, "moe_dispatch_padded: up to 256 experts are supported");
    const int64_t cap = (T * k + 127) / 128 * 128 + 128 * E;
    c10::cuda::CUDAGuard guard(x.device());
    auto iopt = x.options().dtype(at::kInt);
    Tensor offsets = at::empty({E + 1}, iopt), cursor = at::empty({E}, iopt);
    Tensor tile_row0 = at::empty({cap / 128}, iopt), tile_expert = at::empty({cap / 128}, iopt);
    Tensor num_tiles = at::empty({1}, iopt);
    Tensor routed = at::zeros({cap, D}, x.options()), src_row = at::full({cap}, -1, iopt), inv = at::empty({T, k}, iopt);
    fs2::moe_grouped_layout(counts.data_ptr<int>(), static_cast<int>(E), offsets.data_ptr<int>(), cursor.data_ptr<int>(),
                            tile_row0.data_ptr<int>(), tile_expert.data_ptr<int>(), num_tiles.data_ptr<int>(),
                            stream_of(x));
    fs2::moe_dispatch(x.data_ptr(), expert_ids.data_ptr<int>(), gates.data_ptr<float>(), offsets.data_ptr<int>(),
                      cursor.data_ptr<int>(), routed.data_ptr(), src_row.data_ptr<int>(), inv.data_ptr<int>(),
                      static_cast<int>(T), static_cast<int>(k), static_cast<int>(D), scale_by_gate, stream_of(x));
    g_launches += 2;
    return {routed, src_row, inv, offsets, tile_row0, tile_expert, num_tiles};
}

// y [cap, N] = grouped(x [cap, K], w): w is [E, K, N] (`w_kn`) or [E, N, K]; one launch, no host-side sizes.
Tensor grouped_gemm(const Tensor& x, const Tensor& w, bool w_kn, const Tensor& tile_row0, const Tensor& tile_expert,
                    const Tensor& num_tiles) {
    TORCH_CHECK(x.is_cuda() && is_bf16(x) && x.dim() == 2 && x.is_contiguous() && aligned16(x) && is_bf16(w) &&
                    w.dim() == 3 && w.is_contiguous() && aligned16(w),
                "grouped_gemm: x [rows, K] and w [E, ., .] must be contiguous bf16 CUDA tensors");
    const int64_t rows = x.size(0), K = x.size(1), E = w.size(0);
    const int64_t N = w_kn ? w.size(2) : w.size(1);
    TORCH_CHECK((w_kn ? w.size(1) : w.size(2)) == K && K % 8 == 0 && N % 8 == 0 && rows % 128 == 0,
                "grouped_gemm: shape mismatch (K, N multiples of 8; rows a multiple of 128)");
    TORCH_CHECK(tile_row0.scalar_type() == at::kInt && tile_expert.scalar_type() == at::kInt &&
                    num_tiles.scalar_type() == at::kInt && tile_row0.numel() >= rows / 128 &&
                    tile_expert.numel() >= rows / 128 && num_tiles.numel() == 1,
                "grouped_gemm: bad tile tables");
    check_status();
    c10::cuda::CUDAGuard guard(x.device());
    // rows past the last tile (the buffer is sized for the worst case) are never written by the kernel and never read
    // by a consumer: everything downstream is bounded by the same tile tables or indexes rows explicitly
    Tensor y = at::empty({rows, N}, x.options());
    const char* err = fs2::gemm_grouped_bf16_tcgen05(
        x.data_ptr(), w.data_ptr(), y.data_ptr(), static_cast<int>(rows), static_cast<int>(N), static_cast<int>(K), w_kn,
        static_cast<int>(E), tile_row0.data_ptr<int>(), tile_expert.data_ptr<int>(), num_tiles.data_ptr<int>(),
        static_cast<int>(rows / 128), status_dev_ptr(), num_sms(x), stream_of(x));
    TORCH_CHECK(err == nullptr, "grouped_gemm: ", err);
    g_launches += 1;
    return y;
}

// dw [E, M, N] (fp32) = per-expert x^T @ dy over the padded row ranges given by offsets [E + 1].
Tensor grouped_gemm_wgrad(const Tensor& x, const Tensor& dy, const Tensor& offsets) {
    TORCH_CHECK(x.is_cuda() && is_bf16(x) && is_bf16(dy) && x.dim() == 2 && dy.dim() == 2 && x.is_contiguous() &&
                    dy.is_contiguous() && x.size(0) == dy.size(0) && aligned16(x) && aligned16(dy),
                "grouped_gemm_wgrad: x [rows, M] and dy [rows, N] must be contiguous bf16 CUDA matrices");
    const int64_t rows = x.size(0), M = x.size(1), N = dy.size(1), E = offsets.numel() - 1;
    TORCH_CHECK(offsets.scalar_type() == at::kInt && E >= 1 && M % 128 == 0 && N % 8 == 0,
                "grouped_gemm_wgrad: offsets must be int32 [E + 1]; M a multiple of 128, N of 8");
    check_status();
    c10::cuda::CUDAGuard guard(x.device());
    Tensor dw = at::empty({E, M, N}, x.options().dtype(at::kFloat));
    const char* err = fs2::gemm_grouped_wgrad_bf16_tcgen05(x.data_ptr(), dy.data_ptr(), dw.data_ptr(), true,
                                                           static_cast<int>(rows), static_cast<int>(M),
                                                           static_cast<int>(N), static_cast<int>(E),
                                                           offsets.data_ptr<int>(), status_dev_ptr(), num_sms(x),
                                                           stream_of(x));
    TORCH_CHECK(err == nullptr, "grouped_gemm_wgrad: ", err);
    g_launches += 1;
    return dw;
}

// y[t] (+)= sum_j gate[t, j] * routed[inv[t, j]]
void moe_combine(const Tensor& routed, const Tensor& inv, const std::optional<Tensor>& gates, Tensor y,
                 bool accumulate) {
    TORCH_CHECK(routed.is_cuda() && is_bf16(routed) && routed.dim() == 2 && routed.is_contiguous() && is_bf16(y) &&
                    y.is_contiguous() && y.dim() == 2 && y.size(1) == routed.size(1) && y.size(1) % 8 == 0 &&
                    aligned16(routed) && aligned16(y),
                "moe_combine: routed/y must be contiguous bf16 matrices with D % 8 == 0");
    TORCH_CHECK(inv.scalar_type() == at::kInt && inv.is_contiguous() && inv.dim() == 2 && inv.size(0) == y.size(0),
                "moe_combine: inv must be int32 [T, k]");
    const float* gp = nullptr;
    if (gates.has_value()) {
        TORCH_CHECK(gates->scalar_type() == at::kFloat && gates->is_contiguous() && gates->sizes() == inv.sizes(),
                    "moe_combine: gates must be fp32 [T, k]");
        gp = gates->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(y.device());
    fs2::moe_combine(routed.data_ptr(), inv.data_ptr<int>(), gp, y.data_ptr(), static_cast<int>(y.size(0)),
                     static_cast<int>(inv.size(1)), static_cast<int>(y.size(1)), accumulate, stream_of(y));
    g_launches += 1;
}

// ----------------------------------------------------------------- generation
void ngram_repeat_block(const Tensor& seqs, Tensor probs, int64_t n, double ban_value) {
    TORCH_CHECK(seqs.is_cuda() && seqs.scalar_type() == at::kLong && seqs.dim() == 2 && seqs.is_contiguous(),
                "ngram_repeat_block: seqs must be contiguous int64 [N, S]");
    TORCH_CHECK(probs.is_cuda() && probs.scalar_type() == at::kFloat && probs.dim() == 2 && probs.is_contiguous() &&
                    probs.size(0) == seqs.size(0),
                "ngram_repeat_block: probs must be contiguous fp32 [N, V]");
    TORCH_CHECK(n >= 1, "ngram_repeat_block: n must be positive");
    c10::cuda::CUDAGuard guard(probs.device());
    if (seqs.size(1) < n || seqs.size(0) == 0) return;
    fs2::ngram_repeat_block(reinterpret_cast<const long long*>(seqs.data_ptr<int64_t>()), probs.data_ptr<float>(),
                            static_cast<int>(seqs.size(0)), static_cast<int>(seqs.size(1)),
                            static_cast<int>(probs.size(1)), static_cast<int>(n), static_cast<float>(ban_value),
                            stream_of(probs));
    g_launches += 1;
}

Tensor sample_top_p_top_k(const Tensor& probs, const Tensor& uniform, double p, int64_t k) {
    TORCH_CHECK(probs.is_cuda() && probs.scalar_type() == at::kFloat && probs.dim() == 2 && probs.is_contiguous(),
                "sample_top_p_top_k: probs must be contiguous fp32 [N, V]");
    TORCH_CHECK(uniform.is_cuda() && uniform.scalar_type() == at::kFloat && uniform.is_contiguous() &&
                    uniform.numel() == probs.size(0),
                "sample_top_p_top_k: uniform must be fp32 [N]");
    TORCH_CHECK(p > 0.0 && k >= 0, "sample_top_p_top_k: p must be in (0, 1] and k non-negative");
    c10::cuda::CUDAGuard guard(probs.device());
    Tensor out = at::empty({probs.size(0)}, probs.options().dtype(at::kLong));
    if (probs.size(0) == 0) return out;
    fs2::sample_top_p_top_k(probs.data_ptr<float>(), uniform.data_ptr<float>(),
                            reinterpret_cast<long long*>(out.data_ptr<int64_t>()), static_cast<int>(probs.size(0)),
                            static_cast<int>(probs.size(1)), static_cast<float>(p), static_cast<int>(k),
                            stream_of(probs));
    g_launches += 1;
    return out;
}

std::tuple<Tensor, Tensor> beam_topk(const Tensor& lprobs, const Tensor& beam_scores, int64_t k) {
    TORCH_CHECK(lprobs.is_cuda() && lprobs.scalar_type() == at::kFloat && lprobs.dim() == 3 && lprobs.is_contiguous(),
                "beam_topk: lprobs must be contiguous fp32 [N, beams, V]");
    TORCH_CHECK(beam_scores.is_cuda() && beam_scores.scalar_type() == at::kFloat && beam_scores.is_contiguous() &&
                    beam_scores.dim() == 2 && beam_scores.size(0) == lprobs.size(0) &&
                    beam_scores.size(1) == lprobs.size(1),
                "beam_topk: beam_scores must be contiguous fp32 [N, beams]");
    TORCH_CHECK(k >= 1 && k <= 32 && k <= lprobs.size(1) * lprobs.size(2), "beam_topk: k must be in [1, 32]");
    c10::cuda::CUDAGuard guard(lprobs.device());
    Tensor scores = at::empty({lprobs.size(0), k}, lprobs.options());
    Tensor idx = at::empty({lprobs.size(0), k}, lprobs.options().dtype(at::kLong));
    if (lprobs.size(0) == 0) return {scores, idx};
    fs2::beam_topk(lprobs.data_ptr<float>(), beam_scores.data_ptr<float>(), scores.data_ptr<float>(),
                   reinterpret_cast<long long*>(idx.data_ptr<int64_t>()), static_cast<int>(lprobs.size(0)),
                   static_cast<int>(lprobs.size(1)), static_cast<int>(lprobs.size(2)), static_cast<int>(k),
                   stream_of(lprobs));
    g_launches += 1;
    return {scores, idx};
}

// -------------------------------------------------------------- cross-entropy
void ce_fwd_bwd_inplace(Tensor logits, const Tensor& targets, const std::optional<Tensor>& mask, int64_t pad_idx,
                        Tensor loss) {
    TORCH_CHECK(logits.is_cuda() && is_bf16(logits) && logits.dim() == 2 && logits.is_contiguous() &&
                    logits.size(1) % 8 == 0 && aligned16(logits),
                "ce_fwd_bwd_inplace: logits must be contiguous bf16 [rows, V], V % 8 == 0");
    TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0),
                "ce_fwd_bwd_inplace: targets must be int64 [rows]");
    TORCH_CHECK(loss.scalar_type() == at::kFloat && loss.numel() == 1, "ce_fwd_bwd_inplace: loss must be an fp32 scalar");
    const float* mptr = nullptr;
    if (mask.has_value()) {
        TORCH_CHECK(mask->scalar_type() == at::kFloat && mask->is_contiguous() && mask->numel() == logits.size(0),
                    "ce_fwd_bwd_inplace: mask must be fp32 [rows]");
        mptr = mask->data_ptr<float>();
    }
    const int rows = static_cast<int>(logits.size(0));
    if (rows == 0) return;
    c10::cuda::CUDAGuard guard(logits.device());
    Tensor row_loss = at::empty({rows}, logits.options().dtype(at::kFloat));
    fs2::ce_fwd_bwd(logits.data_ptr(), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), mptr,
                    row_loss.data_ptr<float>(), rows, static_cast<int>(logits.size(1)), static_cast<int>(pad_idx),
                    stream_of(logits));
    g_launches += 1;
    loss.add_(row_loss.sum());
}

// ------------------------------------------------------------------ attention
fs2::AttnParams make_attn_params(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& qb, const Tensor& ql,
                                 const Tensor& kb, const Tensor& kl, int64_t max_q, int64_t max_k, bool causal,
                                 double scale) {
    auto check_view = [](const Tensor& t, const char* name) {
        TORCH_CHECK(t.is_cuda() && is_bf16(t) && t.dim() == 3, name, " must be a bf16 [T, heads, D] CUDA tensor");
        TORCH_CHECK(t.stride(2) == 1 && t.stride(1) == t.size(2), name, " must have contiguous heads");
        TORCH_CHECK(t.stride(0) % 8 == 0 && aligned16(t), name, " must be 16-byte aligned");
    };
    check_view(q, "q");
    check_view(k, "k");
    check_view(v, "v");
    TORCH_CHECK(k.sizes() == v.sizes() && q.size(2) == k.size(2), "attention: shape mismatch");
    TORCH_CHECK(q.size(1) % k.size(1) == 0, "attention: H must be a multiple of Hkv");
    for (const Tensor* t : {&qb, &ql, &kb, &kl})
        TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->dim() == 1 && t->stride(0) == 1,
                    "attention: sequence offsets/lengths must be int32 CUDA vectors");
    TORCH_CHECK(qb.numel() == ql.numel() && kb.numel() == kl.numel() && qb.numel() == kb.numel(),
                "attention: inconsistent number of sequences");
    fs2::AttnParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q.data_ptr());
    p.k = static_cast<const __nv_bfloat16*>(k.data_ptr());
    p.v = static_cast<const __nv_bfloat16*>(v.data_ptr());
    p.q_tstride = q.stride(0);
    p.k_tstride = k.stride(0);
    p.v_tstride = v.stride(0);
    p.q_begins = qb.data_ptr<int>();
    p.q_lens = ql.data_ptr<int>();
    p.k_begins = kb.data_ptr<int>();
    p.k_lens = kl.data_ptr<int>();
    p.num_seqs = static_cast<int>(qb.numel());
    p.total_q = static_cast<int>(q.size(0));
    p.total_k = static_cast<int>(k.size(0));
    p.max_q = static_cast<int>(max_q);
    p.max_k = static_cast<int>(max_k);
    p.H = static_cast<int>(q.size(1));
    p.Hkv = static_cast<int>(k.size(1));
    p.D = static_cast<int>(q.size(2));
    p.causal = causal ? 1 : 0;
    p.scale = static_cast<float>(scale);
    return p;
}

// Dropout on the attention probabilities; only the mma.sync kernels implement it.
bool set_attn_dropout(fs2::AttnParams& p, double dropout_p, int64_t seed) {
    TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, "attention: `dropout_p` must be in [0, 1)");
    if (dropout_p == 0.0) return false;
    TORCH_CHECK(p.window == 0, "attention: dropout cannot be combined with a sliding window");
    p.drop_threshold = static_cast<unsigned int>(std::min(4294967295.0, std::max(1.0, dropout_p * 4294967296.0)));
    p.keep_scale = static_cast<float>(1.0 / (1.0 - dropout_p));
    p.seed = static_cast<unsigned long long>(seed);
    return true;
}

std::tuple<Tensor, Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& qb,
                                    const Tensor& ql, const Tensor& kb, const Tensor& kl, int64_t max_q,
                                    int64_t max_k, bool causal, double scale, int64_t window, double dropout_p,
                                    int64_t seed) {
    fs2::AttnParams p = make_attn_params(q, k, v, qb, ql, kb, kl, max_q, max_k, causal, scale);
    TORCH_CHECK(window >= 0 && (window == 0 || (causal && p.D == 128)),
                "attn_fwd: a sliding window needs causal attention with head_dim 128");
    p.window = static_cast<int>(window);
    c10::cuda::CUDAGuard guard(q.device());
    // rows that belong to no sequence (padding) stay zero
    Tensor out = at::zeros({q.size(0), q.size(1), q.size(2)}, q.options());
    Tensor lse = at::full({q.size(1), q.size(0)}, -INFINITY, q.options().dtype(at::kFloat));
    p.o = static_cast<__nv_bfloat16*>(out.data_ptr());
    p.o_tstride = out.stride(0);
    p.lse = lse.data_ptr<float>();
    // head_dim 128 runs on the tcgen05/TMEM kernel; FAIRSEQ2_B200_ATTN=mma selects the mma.sync kernel instead
    static const bool use_tc = []() {
        const char* e = std::getenv("FAIRSEQ2_B200_ATTN");
        return e == nullptr || std::string(e) != "mma";
    }();
    const bool dropout = set_attn_dropout(p, dropout_p, seed);
    const char* err = ((use_tc || p.window > 0) && p.D == 128 && !dropout)
                          ? fs2::attn_forward_tc(p, status_dev_ptr(), stream_of(q))
                          : fs2::attn_forward(p, stream_of(q));
    TORCH_CHECK(err == nullptr, "attn_fwd: ", err);
    g_launches += 1;
    return {out, lse};
}

void attn_bwd_out(const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
                  const Tensor& lse, const Tensor& qb, const Tensor& ql, const Tensor& kb, const Tensor& kl,
                  int64_t max_q, int64_t max_k, bool causal, double scale, Tensor dq, Tensor dk, Tensor dv,
                  int64_t window, double dropout_p, int64_t seed) {
    fs2::AttnParams p = make_attn_params(q, k, v, qb, ql, kb, kl, max_q, max_k, causal, scale);
    TORCH_CHECK(window >= 0 && (window == 0 || (causal && p.D == 128)),
                "attn_bwd: a sliding window needs causal attention with head_dim 128");
    p.window = static_cast<int>(window);
    auto check_view = [](const Tensor& t, const Tensor& like, const char* name) {
        TORCH_CHECK(t.is_cuda() && is_bf16(t) && t.sizes() == like.sizes() && t.stride(2) == 1 &&
                        t.stride(1) == t.size(2) && t.stride(0) % 8 == 0 && aligned16(t),
                    name, " has a bad layout");
    };
    check_view(dout, q, "dout");
    check_view(out, q, "out");
    check_view(dq, q, "dq");
    check_view(dk, k, "dk");
    check_view(dv, v, "dv");
    c10::cuda::CUDAGuard guard(q.device());
    Tensor delta = at::empty({q.size(1), q.size(0)}, q.options().dtype(at::kFloat));
    p.o = static_cast<__nv_bfloat16*>(out.data_ptr());
    p.o_tstride = out.stride(0);
    p.dout = static_cast<const __nv_bfloat16*>(dout.data_ptr());
    p.do_tstride = dout.stride(0);
    p.dq = static_cast<__nv_bfloat16*>(dq.data_ptr());
    p.dk = static_cast<__nv_bfloat16*>(dk.data_ptr());
    p.dv = static_cast<__nv_bfloat16*>(dv.data_ptr());
    p.dq_tstride = dq.stride(0);
    p.dk_tstride = dk.stride(0);
    p.dv_tstride = dv.stride(0);
    p.lse = lse.data_ptr<float>();
    p.delta = delta.data_ptr<float>();
    static const bool use_tc = []() {
        const char* e = std::getenv("FAIRSEQ2_B200_ATTN");
        return e == nullptr || (std::string(e) != "mma" && std::string(e) != "mma_bwd");
    }();
    const bool dropout = set_attn_dropout(p, dropout_p, seed);
    const char* err = ((use_tc || p.window > 0) && p.D == 128 && !dropout)
                          ? fs2::attn_backward_tc(p, status_dev_ptr(), stream_of(q))
                          : fs2::attn_backward(p, stream_of(q));
    TORCH_CHECK(err == nullptr, "attn_bwd: ", err);
    g_launches += 3;
}

std::tuple<Tensor, Tensor, Tensor> attn_bwd(const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v,
                                            const Tensor& out, const Tensor& lse, const Tensor& qb, const Tensor& ql,
                                            const Tensor& kb, const Tensor& kl, int64_t max_q, int64_t max_k,
                                            bool causal, double scale, int64_t window, double dropout_p,
                                            int64_t seed) {
    // tokens outside every sequence (padding) receive zero gradients
    Tensor dq = at::zeros({q.size(0), q.size(1), q.size(2)}, q.options());
    Tensor dk = at::zeros({k.size(0), k.size(1), k.size(2)}, k.options());
    Tensor dv = at::zeros({v.size(0), v.size(1), v.size(2)}, v.options());
    attn_bwd_out(dout, q, k, v, out, lse, qb, ql, kb, kl, max_q, max_k, causal, scale, dq, dk, dv, window, dropout_p,
                 seed);
    return {dq, dk, dv};
}

// ------------------------------------------------------------------ optimizer
// Device-memory copy of the status word that the optimizer kernels read ("skip the update if a collective gave
// up"); one word per device, zero until `refresh_status_guard` finds the status word set.
int* g_guard_dev[64] = {};

int* status_guard_ptr(int device) {
    TORCH_CHECK(device >= 0 && device < 64, "status guard: bad device index");
    if (g_guard_dev[device] == nullptr) {
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
        TORCH_CHECK(cudaMalloc(reinterpret_cast<void**>(&g_guard_dev[device]), sizeof(int)) == cudaSuccess,
                    "status guard: allocation failed");
        TORCH_CHECK(cudaMemset(g_guard_dev[device], 0, sizeof(int)) == cudaSuccess, "status guard: memset failed");
    }
    return g_guard_dev[device];
}

// Once per optimizer step, on the current stream of `device`: the optimizer launches that follow see the status word
// as it is at this point of the stream (after the collectives of the step).
void refresh_status_guard(int64_t device) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    fs2::copy_status(status_dev_ptr(), status_guard_ptr(static_cast<int>(device)),
                     at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream());
    g_launches += 1;
}

void multi_tensor_adamw(const std::vector<Tensor>& masters, const std::vector<Tensor>& grads,
                        const std::vector<Tensor>& ms, const std::vector<Tensor>& vs, const std::vector<Tensor>& lows,
                        double lr, double beta1, double beta2, double eps, double wd, int64_t step,
                        const std::optional<Tensor>& grad_scale) {
    const size_t n = masters.size();
    TORCH_CHECK(grads.size() == n && ms.size() == n && vs.size() == n && lows.size() == n,
                "multi_tensor_adamw: list sizes differ");
    const float* gs = nullptr;
    if (grad_scale.has_value()) {
        TORCH_CHECK(grad_scale->is_cuda() && grad_scale->scalar_type() == at::kFloat && grad_scale->numel() == 1,
                    "multi_tensor_adamw: grad_scale must be an fp32 device scalar");
        gs = grad_scale->data_ptr<float>();
    }
    for (size_t i = 0; i < n; ++i) {
        const Tensor& p = masters[i];
        const Tensor& g = grads[i];
        TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kFloat && p.is_contiguous(), "multi_tensor_adamw: master weights must be contiguous fp32");
        TORCH_CHECK(ms[i].scalar_type() == at::kFloat && vs[i].scalar_type() == at::kFloat && ms[i].is_contiguous() &&
                        vs[i].is_contiguous() && ms[i].numel() == p.numel() && vs[i].numel() == p.numel(),
                    "multi_tensor_adamw: optimizer state must be contiguous fp32 of the parameter's size");
        TORCH_CHECK(g.is_contiguous() && g.numel() == p.numel() && (is_bf16(g) || g.scalar_type() == at::kFloat),
                    "multi_tensor_adamw: gradients must be contiguous bf16/fp32");
        void* low = nullptr;
        if (lows[i].numel() > 0) {
            TORCH_CHECK(is_bf16(lows[i]) && lows[i].is_contiguous() && lows[i].numel() == p.numel() && aligned16(lows[i]),
                        "multi_tensor_adamw: low-precision copies must be contiguous bf16");
            low = lows[i].data_ptr();
        }
        TORCH_CHECK(aligned16(p) && aligned16(g) && aligned16(ms[i]) && aligned16(vs[i]),
                    "multi_tensor_adamw: tensors must be 16-byte aligned");
        c10::cuda::CUDAGuard guard(p.device());
        fs2::adamw(p.data_ptr<float>(), g.data_ptr(), is_bf16(g), ms[i].data_ptr<float>(), vs[i].data_ptr<float>(), low,
                   static_cast<size_t>(p.numel()), static_cast<float>(lr), static_cast<float>(beta1),
                   static_cast<float>(beta2), static_cast<float>(eps), static_cast<float>(wd), static_cast<int>(step),
                   gs, status_guard_ptr(p.get_device()), num_sms(p), stream_of(p));
        g_launches += 1;
    }
}

Tensor multi_tensor_l2_norm_sq(const std::vector<Tensor>& ts) {
    TORCH_CHECK(!ts.empty(), "multi_tensor_l2_norm_sq: empty list");
    c10::cuda::CUDAGuard guard(ts[0].device());
    Tensor out = at::zeros({}, ts[0].options().dtype(at::kFloat));
    for (const Tensor& t : ts) {
        TORCH_CHECK(t.is_cuda() && t.is_contiguous() && (is_bf16(t) || t.scalar_type() == at::kFloat) && aligned16(t),
                    "multi_tensor_l2_norm_sq: tensors must be contiguous, 16-byte aligned bf16/fp32");
        fs2::l2_norm_sq(t.data_ptr(), is_bf16(t), static_cast<size_t>(t.numel()), out.data_ptr<float>(), num_sms(t),
                        stream_of(t));
        g_launches += 1;
    }
    return out;
}

void multi_tensor_scale(const std::vector<Tensor>& ts, const Tensor& scale) {
    TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::kFloat && scale.numel() == 1,
                "multi_tensor_scale: scale must be an fp32 device scalar");
    for (const Tensor& t : ts) {
        TORCH_CHECK(t.is_cuda() && t.is_contiguous() && (is_bf16(t) || t.scalar_type() == at::kFloat) && aligned16(t),
                    "multi_tensor_scale: tensors must be contiguous, 16-byte aligned bf16/fp32");
        c10::cuda::CUDAGuard guard(t.device());
        fs2::scale_inplace(t.data_ptr(), is_bf16(t), static_cast<size_t>(t.numel()), scale.data_ptr<float>(),
                           num_sms(t), stream_of(t));
        g_launches += 1;
    }
}

// ------------------------------------------------------- symmetric-memory comm
fs2::CommPeers make_peers(const std::vector<int64_t>& ptrs, int64_t rank, double wait_limit_s) {
    TORCH_CHECK(!ptrs.empty() && ptrs.size() <= static_cast<size_t>(fs2::kCommMaxRanks),
                "comm: between 1 and ", fs2::kCommMaxRanks, " ranks are supported");
    TORCH_CHECK(rank >= 0 && rank < static_cast<int64_t>(ptrs.size()), "comm: bad rank");
    fs2::CommPeers p{};
    for (size_t i = 0; i < ptrs.size(); ++i) {
        TORCH_CHECK(ptrs[i] != 0 && ptrs[i] % 16 == 0, "comm: peer base pointers must be non-null and 16-byte aligned");
        p.base[i] = reinterpret_cast<void*>(ptrs[i]);
    }
    p.world = static_cast<int>(ptrs.size());
    p.rank = static_cast<int>(rank);
    p.wait_limit_ns = static_cast<unsigned long long>(wait_limit_s * 1e9);
    return p;
}

fs2::CommSegments make_segments(const std::vector<int64_t>& offs, const std::vector<int64_t>& numels) {
    TORCH_CHECK(offs.size() == numels.size() && !offs.empty() &&
                    offs.size() <= static_cast<size_t>(fs2::kCommMaxSegments),
                "comm: between 1 and ", fs2::kCommMaxSegments, " segments are supported");
    fs2::CommSegments s{};
    s.count = static_cast<int>(offs.size());
    for (size_t i = 0; i < offs.size(); ++i) {
        TORCH_CHECK(offs[i] % 8 == 0 && numels[i] % 8 == 0, "comm: segments must be multiples of 8 elements");
        TORCH_CHECK(i == 0 || offs[i] == offs[i - 1] + numels[i - 1], "comm: segments must tile the shard buffer");
        s.off[i] = offs[i];
        s.numel[i] = numels[i];
    }
    return s;
}

void comm_barrier(const std::vector<int64_t>& ptrs, int64_t rank, int64_t slot, int64_t epoch, int64_t device,
                  double wait_limit_s) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    fs2::comm_barrier(make_peers(ptrs, rank, wait_limit_s), static_cast<int>(slot), static_cast<uint32_t>(epoch),
                      status_dev_ptr(), at::cuda::getCurrentCUDAStream(device).stream());
    g_launches += 1;
}

void comm_signal(const std::vector<int64_t>& ptrs, int64_t rank, int64_t slot, int64_t epoch, int64_t device) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    fs2::comm_signal(make_peers(ptrs, rank, 1.0), static_cast<int>(slot), static_cast<uint32_t>(epoch),
                     at::cuda::getCurrentCUDAStream(device).stream());
    g_launches += 1;
}

void comm_allgather_segments(const std::vector<int64_t>& ptrs, int64_t rank, const std::vector<int64_t>& offs,
                             const std::vector<int64_t>& numels, int64_t shard_byte_off, Tensor full, int64_t slot,
                             int64_t epoch, int64_t blocks, double wait_limit_s) {
    TORCH_CHECK(full.is_cuda() && full.is_contiguous() && full.element_size() == 2 && aligned16(full),
                "comm_allgather_segments: `full` must be a contiguous 2-byte CUDA tensor");
    const int64_t shard_numel = offs.back() + numels.back();
    TORCH_CHECK(full.numel() == shard_numel * static_cast<int64_t>(ptrs.size()),
                "comm_allgather_segments: `full` must hold world x shard elements");
    TORCH_CHECK(shard_byte_off % 16 == 0, "comm_allgather_segments: unaligned shard offset");
    c10::cuda::CUDAGuard guard(full.device());
    fs2::comm_allgather_segments(make_peers(ptrs, rank, wait_limit_s), make_segments(offs, numels), shard_byte_off,
                                 full.data_ptr(), shard_numel, static_cast<int>(slot), static_cast<uint32_t>(epoch),
                                 static_cast<int>(blocks), status_dev_ptr(), stream_of(full));
    g_launches += 1;
}

// All-gather of the same segment layout through the copy engines: one peer-to-peer cudaMemcpyAsync per
// (peer, segment), peers visited in ring order starting after this rank so that no GPU is read by everyone at
// once. No SM takes part, so the GEMMs that run next to it on the compute stream keep all of them.
void comm_allgather_copy(const std::vector<int64_t>& ptrs, int64_t rank, const std::vector<int64_t>& offs,
                         const std::vector<int64_t>& numels, int64_t shard_byte_off, Tensor full, int64_t slot,
                         int64_t epoch, double wait_limit_s) {
    TORCH_CHECK(full.is_cuda() && full.is_contiguous() && full.element_size() == 2 && aligned16(full),
                "comm_allgather_copy: `full` must be a contiguous 2-byte CUDA tensor");
    TORCH_CHECK(offs.size() == numels.size() && !offs.empty(), "comm_allgather_copy: bad segment table");
    const int64_t W = static_cast<int64_t>(ptrs.size());
    const int64_t shard_numel = offs.back() + numels.back();
    TORCH_CHECK(full.numel() == shard_numel * W, "comm_allgather_copy: `full` must hold world x shard elements");
    c10::cuda::CUDAGuard guard(full.device());
    cudaStream_t st = stream_of(full);
    if (epoch != 0) {
        fs2::comm_wait(make_peers(ptrs, rank, wait_limit_s), static_cast<int>(slot), static_cast<uint32_t>(epoch),
                       status_dev_ptr(), st);
        g_launches += 1;
    }
    char* dst = static_cast<char*>(full.data_ptr());
    for (int64_t k = 1; k <= W; ++k) {
        const int64_t r = (rank + k) % W;                       // own shard last: it needs no link
        const char* src = reinterpret_cast<const char*>(ptrs[static_cast<size_t>(r)]) + shard_byte_off;
        for (size_t i = 0; i < offs.size(); ++i) {
            const size_t bytes = static_cast<size_t>(numels[i]) * 2;
            C10_CUDA_CHECK(cudaMemcpyAsync(dst + (W * offs[i] + r * numels[i]) * 2, src + offs[i] * 2, bytes,
                                           cudaMemcpyDeviceToDevice, st));
        }
    }
}

// Vocabulary-parallel lookup whose rows go straight to the ranks that own the tokens (no reduce-scatter).
void embed_push(const std::vector<int64_t>& ptrs, int64_t rank, const Tensor& ids, const Tensor& table, int64_t lo,
                int64_t out_byte_off, int64_t rows_per_rank, double wait_limit_s) {
    TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && table.is_cuda() &&
                    is_bf16(table) && table.dim() == 2 && table.is_contiguous() && table.size(1) % 8 == 0 &&
                    aligned16(table),
                "embed_push: ids must be int64, the table shard a contiguous bf16 [rows, D] with D % 8 == 0");
    TORCH_CHECK(out_byte_off % 16 == 0 && rows_per_rank > 0 &&
                    ids.numel() == rows_per_rank * static_cast<int64_t>(ptrs.size()),
                "embed_push: the tokens must split evenly over the ranks and the output offset be 16-byte aligned");
    c10::cuda::CUDAGuard guard(table.device());
    fs2::embed_push(make_peers(ptrs, rank, wait_limit_s), reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()),
                    table.data_ptr(), lo, table.size(0), out_byte_off, ids.numel(), static_cast<int>(table.size(1)),
                    rows_per_rank, stream_of(table));
    g_launches += 1;
}

Tensor embed_pull_bwd(const std::vector<int64_t>& ptrs, int64_t rank, const Tensor& ids, int64_t dout_byte_off,
                      int64_t rows, int64_t D, int64_t lo, int64_t rows_per_rank, double wait_limit_s) {
    TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "embed_pull_bwd: bad ids");
    TORCH_CHECK(dout_byte_off % 16 == 0 && D % 8 == 0 && rows_per_rank > 0 &&
                    ids.numel() == rows_per_rank * static_cast<int64_t>(ptrs.size()),
                "embed_pull_bwd: bad layout");
    c10::cuda::CUDAGuard guard(ids.device());
    Tensor dtable = at::zeros({rows, D}, ids.options().dtype(at::kFloat));
    fs2::embed_pull_bwd(make_peers(ptrs, rank, wait_limit_s),
                        reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), dout_byte_off,
                        dtable.data_ptr<float>(), lo, rows, ids.numel(), static_cast<int>(D), rows_per_rank,
                        stream_of(ids));
    g_launches += 1;
    return dtable;
}

// Device scalar that receives a sum of squares, or null.
float* norm_out_ptr(const std::optional<Tensor>& norm_out, const Tensor& like) {
    if (!norm_out.has_value()) return nullptr;
    TORCH_CHECK(norm_out->is_cuda() && norm_out->scalar_type() == at::kFloat && norm_out->numel() == 1 &&
                    norm_out->device() == like.device(),
                "comm: `norm_out` must be an fp32 scalar on the device of the output");
    return norm_out->data_ptr<float>();
}

void comm_reducescatter_segments(const std::vector<int64_t>& ptrs, int64_t rank, const std::vector<int64_t>& offs,
                                 const std::vector<int64_t>& numels, int64_t full_byte_off, Tensor out, double scale,
                                 bool accumulate, int64_t slot, int64_t epoch, int64_t blocks, double wait_limit_s,
                                 const std::optional<Tensor>& norm_out) {
    const int64_t shard_numel = offs.back() + numels.back();
    float* norm_ptr = norm_out_ptr(norm_out, out);
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() == shard_numel && aligned16(out) &&
                    (out.scalar_type() == at::kFloat || is_bf16(out)),
                "comm_reducescatter_segments: `out` must be a contiguous fp32/bf16 shard-sized CUDA tensor");
    TORCH_CHECK(full_byte_off % 16 == 0, "comm_reducescatter_segments: unaligned offset");
    c10::cuda::CUDAGuard guard(out.device());
    fs2::comm_reducescatter_segments(make_peers(ptrs, rank, wait_limit_s), make_segments(offs, numels),
                                     full_byte_off, out.data_ptr(), out.scalar_type() == at::kFloat, shard_numel,
                                     static_cast<float>(scale), accumulate, static_cast<int>(slot),
                                     static_cast<uint32_t>(epoch), static_cast<int>(blocks), norm_ptr,
                                     status_dev_ptr(), stream_of(out));
    g_launches += 1;
}

// Reduce-scatter whose NVLink half runs on the copy engines: after the barrier that says every rank's gradients of
// this unit are final, the peers' slices of the local shard are copied into `staging` ([W - 1, shard] bf16, local
// memory), then one short kernel sums them with the own slice in fp32. The SMs are busy for a local-memory pass only.
void comm_reducescatter_copy(const std::vector<int64_t>& ptrs, int64_t rank, const std::vector<int64_t>& offs,
                             const std::vector<int64_t>& numels, int64_t full_byte_off, Tensor staging, Tensor out,
                             double scale, bool accumulate, int64_t slot, int64_t epoch, int64_t blocks,
                             double wait_limit_s, const std::optional<Tensor>& norm_out) {
    const int64_t W = static_cast<int64_t>(ptrs.size());
    const int64_t shard_numel = offs.back() + numels.back();
    float* norm_ptr = norm_out_ptr(norm_out, out);
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() == shard_numel && aligned16(out) &&
                    (out.scalar_type() == at::kFloat || is_bf16(out)),
                "comm_reducescatter_copy: `out` must be a contiguous fp32/bf16 shard-sized CUDA tensor");
    TORCH_CHECK(staging.is_cuda() && staging.is_contiguous() && is_bf16(staging) && aligned16(staging) &&
                    staging.numel() >= (W - 1) * shard_numel,
                "comm_reducescatter_copy: `staging` must be a contiguous bf16 CUDA tensor of (world - 1) shards");
    TORCH_CHECK(full_byte_off % 16 == 0, "comm_reducescatter_copy: unaligned offset");
    c10::cuda::CUDAGuard guard(out.device());
    cudaStream_t st = stream_of(out);
    const auto peers = make_peers(ptrs, rank, wait_limit_s);
    const auto segs = make_segments(offs, numels);
    fs2::comm_barrier(peers, static_cast<int>(slot), static_cast<uint32_t>(epoch), status_dev_ptr(), st);
    char* stage = static_cast<char*>(staging.data_ptr());
    const void* staged[8];
    for (int64_t k = 1; k < W; ++k) {
        const int64_t r = (rank + k) % W;
        const char* src = reinterpret_cast<const char*>(ptrs[static_cast<size_t>(r)]) + full_byte_off;
        char* dst = stage + (k - 1) * shard_numel * 2;
        staged[k - 1] = dst;
        for (size_t i = 0; i < offs.size(); ++i) {
            C10_CUDA_CHECK(cudaMemcpyAsync(dst + offs[i] * 2, src + (W * offs[i] + rank * numels[i]) * 2,
                                           static_cast<size_t>(numels[i]) * 2, cudaMemcpyDeviceToDevice, st));
        }
    }
    const char* own = reinterpret_cast<const char*>(ptrs[static_cast<size_t>(rank)]) + full_byte_off;
    fs2::comm_reduce_staged(own, staged, static_cast<int>(W - 1), segs, static_cast<int>(rank), static_cast<int>(W),
                            out.data_ptr(), out.scalar_type() == at::kFloat, static_cast<float>(scale), accumulate,
                            static_cast<int>(blocks), norm_ptr, st);
    g_launches += 2;
}

void comm_reducescatter_adamw(const std::vector<int64_t>& ptrs, int64_t rank, const std::vector<int64_t>& offs,
                              const std::vector<int64_t>& numels, int64_t full_byte_off, Tensor master, Tensor m,
                              Tensor v, const std::optional<Tensor>& low, double scale, double lr, double beta1,
                              double beta2, double eps, double wd, int64_t step, int64_t slot, int64_t epoch,
                              int64_t blocks, double wait_limit_s, const std::optional<Tensor>& grad_scale) {
    const float* scale_ptr = nullptr;
    if (grad_scale.has_value()) {
        TORCH_CHECK(grad_scale->is_cuda() && grad_scale->scalar_type() == at::kFloat && grad_scale->numel() == 1 &&
                        grad_scale->device() == master.device(),
                    "comm_reducescatter_adamw: grad_scale must be an fp32 scalar on the device of the shard");
        scale_ptr = grad_scale->data_ptr<float>();
    }
    const int64_t shard_numel = offs.back() + numels.back();
    for (const Tensor* t : {&master, &m, &v})
        TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kFloat &&
                        t->numel() == shard_numel && aligned16(*t),
                    "comm_reducescatter_adamw: master/m/v must be contiguous fp32 shard-sized CUDA tensors");
    void* lowp = nullptr;
    if (low.has_value()) {
        TORCH_CHECK(low->is_cuda() && low->is_contiguous() && is_bf16(*low) && low->numel() == shard_numel &&
                        aligned16(*low),
                    "comm_reducescatter_adamw: `low` must be a contiguous bf16 shard-sized CUDA tensor");
        lowp = low->data_ptr();
    }
    TORCH_CHECK(full_byte_off % 16 == 0 && step >= 1, "comm_reducescatter_adamw: bad argument");
    c10::cuda::CUDAGuard guard(master.device());
    fs2::comm_reducescatter_adamw(make_peers(ptrs, rank, wait_limit_s), make_segments(offs, numels), full_byte_off,
                                  master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), lowp,
                                  static_cast<float>(scale), static_cast<float>(lr), static_cast<float>(beta1),
                                  static_cast<float>(beta2), static_cast<float>(eps), static_cast<float>(wd),
                                  static_cast<int>(step), scale_ptr, static_cast<int>(slot),
                                  static_cast<uint32_t>(epoch), static_cast<int>(blocks), status_dev_ptr(),
                                  stream_of(master));
    g_launches += 1;
}

void comm_allreduce_f32(const std::vector<int64_t>& ptrs, int64_t rank, int64_t byte_off, Tensor out, int64_t op,
                        int64_t slot, int64_t epoch, double wait_limit_s) {
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == at::kFloat,
                "comm_allreduce_f32: `out` must be a contiguous fp32 CUDA tensor");
    TORCH_CHECK(byte_off % 16 == 0 && op >= 0 && op <= 4, "comm_allreduce_f32: bad argument");
    c10::cuda::CUDAGuard guard(out.device());
    const int64_t n = out.numel();
    const int blocks = static_cast<int>(std::min<int64_t>(std::max<int64_t>((n + 255) / 256, 1), 64));
    fs2::comm_allreduce_f32(make_peers(ptrs, rank, wait_limit_s), byte_off, out.data_ptr<float>(), n,
                            static_cast<int>(op), static_cast<int>(slot), static_cast<uint32_t>(epoch), blocks,
                            status_dev_ptr(), stream_of(out));
    g_launches += 1;
}

void comm_allreduce_inplace(const std::vector<int64_t>& ptrs, int64_t rank, int64_t byte_off, int64_t numel, bool f32,
                            double scale, int64_t slot_in, int64_t slot_mid, int64_t epoch, int64_t counter_byte_off,
                            int64_t device, int64_t blocks, double wait_limit_s) {
    const int64_t per = f32 ? 4 : 8;
    TORCH_CHECK(byte_off % 16 == 0 && numel % per == 0 && numel > 0, "comm_allreduce_inplace: the bucket must be a "
                "whole number of 16-byte vectors at a 16-byte aligned offset");
    TORCH_CHECK(counter_byte_off % 8 == 0 && blocks >= 1 && blocks <= 148 && epoch >= 1,
                "comm_allreduce_inplace: bad argument (the counter is two words, 8-byte aligned; epochs start at 1)");
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    auto* counter = reinterpret_cast<unsigned int*>(ptrs[static_cast<size_t>(rank)] + counter_byte_off);
    fs2::comm_allreduce_inplace(make_peers(ptrs, rank, wait_limit_s), byte_off, numel, f32, static_cast<float>(scale),
                                static_cast<int>(slot_in), static_cast<int>(slot_mid), static_cast<uint32_t>(epoch),
                                counter, static_cast<int>(blocks), status_dev_ptr(),
                                at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream());
    g_launches += 1;
}

void comm_allreduce_multimem(const std::vector<int64_t>& ptrs, int64_t rank, int64_t multicast_ptr, int64_t byte_off,
                             int64_t numel, bool f32, double scale, int64_t slot_in, int64_t slot_out, int64_t epoch,
                             int64_t counter_byte_off, int64_t device, int64_t blocks, double wait_limit_s) {
    const int64_t per = f32 ? 4 : 8;
    TORCH_CHECK(multicast_ptr != 0, "comm_allreduce_multimem: the arena has no multicast mapping");
    TORCH_CHECK(byte_off % 16 == 0 && numel > 0 && numel % per == 0 && counter_byte_off % 4 == 0 && blocks > 0,
                "comm_allreduce_multimem: the buffer must be 16-byte aligned and a multiple of 16 bytes");
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    auto* counter = reinterpret_cast<unsigned int*>(ptrs[static_cast<size_t>(rank)] + counter_byte_off);
    fs2::comm_allreduce_multimem(make_peers(ptrs, rank, wait_limit_s), reinterpret_cast<void*>(multicast_ptr), byte_off,
                                 numel, f32, static_cast<float>(scale), static_cast<int>(slot_in),
                                 static_cast<int>(slot_out), static_cast<uint32_t>(epoch), counter,
                                 static_cast<int>(blocks), status_dev_ptr(),
                                 at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream());
    g_launches += 1;
}

void comm_pull(const std::vector<int64_t>& ptrs, int64_t rank, int64_t src_rank, int64_t byte_off, Tensor dst,
               int64_t slot, int64_t epoch, double wait_limit_s) {
    TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && aligned16(dst) && (dst.numel() * dst.element_size()) % 16 == 0,
                "comm_pull: `dst` must be contiguous, 16-byte aligned and a multiple of 16 bytes");
    TORCH_CHECK(src_rank >= 0 && src_rank < static_cast<int64_t>(ptrs.size()) && byte_off % 16 == 0, "comm_pull: bad argument");
    c10::cuda::CUDAGuard guard(dst.device());
    const int64_t bytes = dst.numel() * dst.element_size();
    const int blocks = static_cast<int>(std::min<int64_t>(std::max<int64_t>(bytes / (512 * 16 * 4), 1), 32));
    fs2::comm_pull(make_peers(ptrs, rank, wait_limit_s), static_cast<int>(src_rank), byte_off, dst.data_ptr(), bytes,
                   static_cast<int>(slot), static_cast<uint32_t>(epoch), blocks, status_dev_ptr(), stream_of(dst));
    g_launches += 1;
}

void comm_alltoall(const std::vector<int64_t>& ptrs, int64_t rank, int64_t byte_off, Tensor dst,
                   const Tensor& send_offs, int64_t slot, int64_t epoch, double wait_limit_s) {
    TORCH_CHECK(dst.is_cuda() && dst.is_contiguous(), "comm_alltoall: `dst` must be a contiguous CUDA tensor");
    const int64_t W = static_cast<int64_t>(ptrs.size());
    TORCH_CHECK(send_offs.is_cuda() && send_offs.scalar_type() == at::kLong && send_offs.is_contiguous() &&
                    send_offs.numel() == W * (W + 1),
                "comm_alltoall: `send_offs` must be an int64 [W, W + 1] CUDA tensor");
    c10::cuda::CUDAGuard guard(dst.device());
    const int64_t row = dst.dim() > 1 ? dst.numel() / std::max<int64_t>(dst.size(0), 1) : 1;
    fs2::comm_alltoall(make_peers(ptrs, rank, wait_limit_s), byte_off, dst.data_ptr(),
                       reinterpret_cast<const long long*>(send_offs.data_ptr<int64_t>()),
                       static_cast<int>(row * dst.element_size()), static_cast<int>(slot),
                       static_cast<uint32_t>(epoch), 8, status_dev_ptr(), stream_of(dst));
    g_launches += 1;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "fairseq2_b200 sm_100a kernels";
    m.def("gemm_bf16", &gemm_bf16);
    m.def("gemm_reduce_scatter", &gemm_reduce_scatter);
    m.def("gemm_bf16_view", &gemm_bf16_view);
    m.def("gemm_allgather", &gemm_allgather);
    m.def("gemm_scatter", &gemm_scatter);
    m.def("reduce_slices", &reduce_slices);
    m.def("rms_norm_fwd", &rms_norm_fwd);
    m.def("rms_norm_bwd", &rms_norm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("rstd"),
          py::arg("dres") = std::nullopt);
    m.def("add_rms_norm_fwd", &add_rms_norm_fwd);
    m.def("layer_norm_fwd", &layer_norm_fwd, py::arg("x"), py::arg("w"), py::arg("b"), py::arg("eps"),
          py::arg("gelu") = false);
    m.def("layer_norm_bwd", &layer_norm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("mean"),
          py::arg("rstd"), py::arg("b_for_gelu") = std::nullopt);
    m.def("swiglu_fwd", &swiglu_fwd);
    m.def("swiglu_bwd", &swiglu_bwd);
    m.def("swiglu2_fwd", &swiglu2_fwd, py::arg("g"), py::arg("u"), py::arg("num_tiles") = std::nullopt);
    m.def("swiglu2_bwd", &swiglu2_bwd, py::arg("dy"), py::arg("g"), py::arg("u"), py::arg("num_tiles") = std::nullopt);
    m.def("copy_rows_bounded", &copy_rows_bounded, py::arg("dst"), py::arg("src"), py::arg("num_tiles") = std::nullopt);
    m.def("rope_inplace", &rope_inplace);
    m.def("ce_fwd_bwd_inplace", &ce_fwd_bwd_inplace);
    m.def("attn_fwd", &attn_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("q_begins"), py::arg("q_lens"),
          py::arg("k_begins"), py::arg("k_lens"), py::arg("max_q"), py::arg("max_k"), py::arg("causal"),
          py::arg("scale"), py::arg("window"), py::arg("dropout_p") = 0.0, py::arg("seed") = 0);
    m.def("attn_bwd", &attn_bwd, py::arg("dout"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"),
          py::arg("lse"), py::arg("q_begins"), py::arg("q_lens"), py::arg("k_begins"), py::arg("k_lens"),
          py::arg("max_q"), py::arg("max_k"), py::arg("causal"), py::arg("scale"), py::arg("window"),
          py::arg("dropout_p") = 0.0, py::arg("seed") = 0);
    m.def("attn_bwd_out", &attn_bwd_out, py::arg("dout"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"),
          py::arg("lse"), py::arg("q_begins"), py::arg("q_lens"), py::arg("k_begins"), py::arg("k_lens"),
          py::arg("max_q"), py::arg("max_k"), py::arg("causal"), py::arg("scale"), py::arg("dq"), py::arg("dk"),
          py::arg("dv"), py::arg("window"), py::arg("dropout_p") = 0.0, py::arg("seed") = 0);
    m.def("multi_tensor_adamw", &multi_tensor_adamw);
    m.def("refresh_status_guard", &refresh_status_guard);
    m.def("multi_tensor_l2_norm_sq", &multi_tensor_l2_norm_sq);
    m.def("multi_tensor_scale", &multi_tensor_scale);
    m.def("comm_barrier", &comm_barrier);
    m.def("comm_signal", &comm_signal);
    m.def("comm_allgather_segments", &comm_allgather_segments);
    m.def("comm_allgather_copy", &comm_allgather_copy);
    m.def("comm_reducescatter_segments", &comm_reducescatter_segments, py::arg("ptrs"), py::arg("rank"),
          py::arg("offs"), py::arg("numels"), py::arg("full_byte_off"), py::arg("out"), py::arg("scale"),
          py::arg("accumulate"), py::arg("slot"), py::arg("epoch"), py::arg("blocks"), py::arg("wait_limit_s"),
          py::arg("norm_out") = std::nullopt);
    m.def("comm_reducescatter_copy", &comm_reducescatter_copy, py::arg("ptrs"), py::arg("rank"), py::arg("offs"),
          py::arg("numels"), py::arg("full_byte_off"), py::arg("staging"), py::arg("out"), py::arg("scale"),
          py::arg("accumulate"), py::arg("slot"), py::arg("epoch"), py::arg("blocks"), py::arg("wait_limit_s"),
          py::arg("norm_out") = std::nullopt);
    m.def("comm_reducescatter_adamw", &comm_reducescatter_adamw, py::arg("ptrs"), py::arg("rank"), py::arg("offs"),
          py::arg("numels"), py::arg("full_byte_off"), py::arg("master"), py::arg("m"), py::arg("v"), py::arg("low"),
          py::arg("scale"), py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("wd"),
          py::arg("step"), py::arg("slot"), py::arg("epoch"), py::arg("blocks"), py::arg("wait_limit_s"),
          py::arg("grad_scale") = std::nullopt);
    m.def("comm_allreduce_f32", &comm_allreduce_f32);
    m.def("comm_allreduce_inplace", &comm_allreduce_inplace);
    m.def("comm_allreduce_multimem", &comm_allreduce_multimem);
    m.def("comm_pull", &comm_pull);
    m.def("embed_push", &embed_push);
    m.def("embed_pull_bwd", &embed_pull_bwd);
    m.def("comm_alltoall", &comm_alltoall);
    m.def("moe_route", &moe_route);
    m.def("moe_dispatch", &moe_dispatch);
    m.def("moe_combine", &moe_combine);
    m.def("embed_vocab_parallel_fwd", &embed_vocab_parallel_fwd);
    m.def("embed_vocab_parallel_bwd", &embed_vocab_parallel_bwd);
    m.def("moe_dispatch_padded", &moe_dispatch_padded);
    m.def("grouped_gemm", &grouped_gemm);
    m.def("grouped_gemm_wgrad", &grouped_gemm_wgrad);
    m.def("w2v_contrastive_fwd", &w2v_contrastive_fwd);
    m.def("w2v_contrastive_bwd", &w2v_contrastive_bwd);
    m.def("w2v_first_conv_supported", &w2v_first_conv_supported);
    m.def("w2v_first_conv_fwd", &w2v_first_conv_fwd);
    m.def("w2v_first_conv_bwd", &w2v_first_conv_bwd);
    m.def("w2v_quantize_fwd", &w2v_quantize_fwd);
    m.def("w2v_quantize_bwd", &w2v_quantize_bwd);
    m.def("moe_ep_layout", &moe_ep_layout);
    m.def("moe_ep_push", &moe_ep_push, py::arg("ptrs"), py::arg("rank"), py::arg("x"), py::arg("expert_ids"),
          py::arg("gates"), py::arg("send_base"), py::arg("cursor"), py::arg("inbox_byte_off"), py::arg("dest"),
          py::arg("E"), py::arg("cap"), py::arg("limit") = std::nullopt, py::arg("dropped") = std::nullopt);
    m.def("moe_ep_layout_padded", &moe_ep_layout_padded);
    m.def("moe_ep_pull", &moe_ep_pull);
    m.def("ngram_repeat_block", &ngram_repeat_block);
    m.def("sample_top_p_top_k", &sample_top_p_top_k);
    m.def("beam_topk", &beam_topk);
    m.def("launch_count", &launch_count);
    m.def("reset_launch_count", &reset_launch_count);
    m.def("check_status", &check_status, "Raises if a kernel recorded a bounded-wait failure.");
    m.def("read_status", &read_status);
    m.def("reset_status", &reset_status);
}
