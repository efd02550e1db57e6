// Internal interface between the dispatcher (api.cu) and the weight-only int4 kernels.
#pragma once

#include "common.cuh"

namespace zt {

struct WoqSkinnyPlan {
  int mt;      // 8-row activation blocks held per CTA (1, 2, 4 or 8)
  int kslice;  // k handled by one CTA
  int nsplit;  // number of K-slices
  size_t partial_bytes;
};

struct WoqStreamPlan {
  int mt;      // 8-row activation blocks (1: M <= 8, 2: M <= 16)
  int r;       // kernel shape index: 0 = 16, 1 = 32, 2 = 64 columns per CTA
  int kslice;  // k handled by one CTA
  int nsplit;  // number of K-slices
  size_t partial_bytes;
};

// Decode kernel (M <= 16).
WoqStreamPlan woq_stream_plan(int64_t M, int64_t N, int64_t K);
bool woq_stream_supported(const zt_woq_linear_args_t &a);
int woq_stream_launch(const zt_woq_linear_args_t &a, cudaStream_t st);

// Decode kernel (M <= 16), bulk-copy staged and work-balanced; needs the fixed scratch below.
size_t woq_streamk_workspace_bytes();
bool woq_streamk_supported(const zt_woq_linear_args_t &a);
int woq_streamk_launch(const zt_woq_linear_args_t &a, cudaStream_t st);

// Mid-size M (17..64 per launch) on mma.sync, weights re-read once per 64 rows.
WoqSkinnyPlan woq_skinny_plan(int64_t M, int64_t N, int64_t K);
bool woq_skinny_supported(const zt_woq_linear_args_t &a);
int woq_skinny_launch(const zt_woq_linear_args_t &a, bool fold, cudaStream_t st);

int woq_generic_launch(const zt_woq_linear_args_t &a, cudaStream_t st);

size_t woq_tcgen05_workspace_bytes(int64_t M, int64_t N, int64_t K);  // fp32 partial sums of its split-K form
bool woq_tcgen05_supported(const zt_woq_linear_args_t &a);
int woq_tcgen05_launch(const zt_woq_linear_args_t &a, cudaStream_t st);
int woq_tcgen05_grouped_launch(const void *x, int64_t total_rows, int64_t N, int64_t K, const int32_t *wq,
                               const void *scales, int scale_dtype, int64_t n_groups, int num_experts, void *y,
                               const int *tile_count, const int4 *tiles, int max_row_tiles, int bt, cudaStream_t st);

}  // namespace zt
