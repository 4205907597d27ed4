// Host launchers of the bandwidth-bound kernels in elementwise.cu.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>

namespace fs2 {

int norm_bwd_grid(int rows, int num_sms);

// `res`/`sum_out` (both or neither): y = rms_norm(x + res) and sum_out = x + res in one pass.
void rms_norm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int D, float eps, bool bf16,
                  int num_sms, cudaStream_t st, const void* res = nullptr, void* sum_out = nullptr);
// `dres` (may be null) is added to dx: the gradient that reaches the normalised tensor through a residual path.
void rms_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_part,
                  float* dw, int rows, int D, bool bf16, int num_sms, cudaStream_t st, const void* dres = nullptr);
// `gelu` (bf16 only): y = gelu(layer_norm(x)) in one pass; the backward then takes the bias as `b_for_gelu` to
// rebuild the pre-activation and treats `dy` as the gradient of the GELU output.
void layer_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows, int D,
                    float eps, bool bf16, int num_sms, cudaStream_t st, bool gelu = false);
void layer_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                    float* dw_part, float* db_part, float* dw, float* db, int rows, int D, bool bf16, int num_sms,
                    cudaStream_t st, const void* b_for_gelu = nullptr);
// Vocabulary-parallel embedding shard [rows, D] covering ids [lo, lo + rows): forward writes the row (times `scale`)
// or zeros; backward accumulates `scale * dout` into an fp32 [rows, D] buffer. D a multiple of 8.
void embed_vocab_parallel_fwd(const long long* ids, const void* table, void* out, size_t tokens, int D, long long lo,
                              long long rows, float scale, cudaStream_t st);
void embed_vocab_parallel_bwd(const long long* ids, const void* dout, float* dtable, size_t tokens, int D, long long lo,
                              long long rows, float scale, cudaStream_t st);
void swiglu_fwd(const void* gu, void* y, size_t rows, int F, int num_sms, cudaStream_t st);
void swiglu_bwd(const void* dy, const void* gu, void* dgu, size_t rows, int F, int num_sms, cudaStream_t st);
// SwiGLU on separate gate / up operands [rows, F]; `num_tiles` (device int, may be null) bounds the rows that hold
// data to num_tiles[0] * 128. Same bound for the row copy (`row_bytes` a multiple of 16).
void swiglu2_fwd(const void* g, const void* u, void* y, size_t rows, int F, const int* num_tiles, int num_sms,
                 cudaStream_t st);
void swiglu2_bwd(const void* dy, const void* g, const void* u, void* dg, void* du, size_t rows, int F,
                 const int* num_tiles, int num_sms, cudaStream_t st);
void copy_rows_bounded(void* dst, const void* src, size_t rows, size_t row_bytes, const int* num_tiles, int num_sms,
                       cudaStream_t st);

void rope_inplace(void* x, const float* freqs, const int* pos, size_t tokens, int heads, int D, size_t tstride,
                  size_t hstride, int max_pos, bool inverse, int num_sms, cudaStream_t st);
void ce_fwd_bwd(void* logits, const long long* targets, const float* mask, float* row_loss, int rows, int V,
                int pad_idx, cudaStream_t st);
// `guard` (may be null): a device-readable status word; the update is skipped when it is non-zero.
void adamw(float* p, const void* g, bool g_bf16, float* m, float* v, void* low, size_t n, float lr, float beta1,
           float beta2, float eps, float wd, int step, const float* grad_scale, const int* guard, int num_sms,
           cudaStream_t st);
// Copies the host-mapped status word into a device-memory word (the `guard` of `adamw`).
void copy_status(const int* host_mapped_status, int* device_guard, cudaStream_t st);
void l2_norm_sq(const void* x, bool bf16, size_t n, float* out, int num_sms, cudaStream_t st);
void scale_inplace(void* x, bool bf16, size_t n, const float* scale, int num_sms, cudaStream_t st);

}  // namespace fs2
