// Argument blocks and host-side launchers shared between the kernel files and the C ABI.
#pragma once

#include "common.cuh"

namespace aq
{
int pymo_per_tensor(const float* in, float* out, int64_t n, float mn, float mx, float delta, float offset,
                    int codes_only, float shift, cudaStream_t st);
int pymo_per_channel(const float* in, float* out, int64_t n, int64_t num_ch, int64_t inner, const float* enc_min,
                     const float* enc_max, const float* enc_delta, const float* enc_offset, float num_steps,
                     int derive, cudaStream_t st);
int v2_minmax_encode(const float* batch, float* running, int running_valid, int dtype, int64_t count, double num_steps,
                     int symmetric, double qmin, float* out, cudaStream_t st);
int fp16_qdq(const float* in, float* out, int64_t n, cudaStream_t st);
int packed_quantize(const float* in, void* out, int64_t n, double e_min, double e_max, double delta, double offset, int bw,
                    int to_signed, cudaStream_t st);
int packed_dequantize(const void* in, float* out, int64_t n, double delta, double offset, int bw, int is_signed,
                      cudaStream_t st);
struct BroadcastArgs
{
    const float* in;
    float* out;
    int64_t n;
    int ndims;
    int64_t in_strides[8];
    int64_t enc_strides[8];
    uint64_t in_m64[8];   // magic64(in_strides[d]) (0 for stride 1): exact 32-bit division by one multiply-high
    const float *mn, *mx, *dl, *of;
};
int pymo_broadcast(const BroadcastArgs& a, cudaStream_t st);
struct V2Args
{
    const void* x;
    void* y;
    uint8_t* mask;
    int64_t n;
    const float* scale;
    const float* offset;
    float qmin, qmax;
    double qmin_wide, qmax_wide;   // the same bounds for the float64 form (grids of 2^24 steps or more)
    int out_kind;
    int dequant_only;
    int wide_ok;   // x and y are 32-byte aligned (set by the launcher): adjacent packets may move as one 32-byte access
    ChanGeom geom;
};
int v2_launch(V2Args a, int dtype, int narrow_internal, cudaStream_t st);
int v2_backward(const void* g, const uint8_t* mask, void* dx, int dtype, int64_t n, cudaStream_t st);
struct V2GradArgs
{
    const void* x;
    const void* grad;
    const uint8_t* mask;
    float* dscale;    // may be null
    float* doffset;   // may be null
    int64_t n;
    const float* scale;
    const float* offset;
    float qmin, qmax;
    ChanGeom geom;
};
int v2_param_grad(V2GradArgs a, int dtype, int reduce, cudaStream_t st);
struct SteArgs
{
    const float* x;
    const float* g;
    float* dx;
    int64_t n;
    const float* enc_min;
    const float* enc_max;
    ChanGeom geom;
};
int ste_v1(SteArgs a, cudaStream_t st);
int64_t minmax_workspace_bytes(int64_t n, int64_t num_ch, int64_t inner);
int minmax_dispatch(const void* x, int dtype, int64_t n, int64_t num_ch, int64_t inner, float* out_min,
                    float* out_max, int propagate_nan, int accumulate, void* ws, int64_t ws_bytes, cudaStream_t st);
int minmax_static(const void* x, int dtype, int64_t n, int64_t num_ch, int64_t inner, float* out_min, float* out_max,
                  int propagate_nan, cudaStream_t st);
int tfe_init_grid(const float* minmax, aq_tfe_state_t* st, cudaStream_t stream);
int tfe_histogram(const float* x, int64_t n, const aq_tfe_state_t* st, uint32_t* hist, int64_t* count,
                  const int32_t* gate, cudaStream_t stream);
int tfe_histogram_many(const float* const* xs, const int64_t* ns, int m, int64_t row_stride, const aq_tfe_state_t* st,
                       uint32_t* hist, int64_t* count, const int32_t* gate, cudaStream_t stream);
int tfe_offer_grid(const float* x, int64_t n, aq_tfe_state_t* st, float* range, int init, void* ws, int64_t ws_bytes,
                   cudaStream_t stream);
int tfe_select_grid(const float* ranges, int num_ranks, int rank, aq_tfe_state_t* st, int32_t* gate,
                    cudaStream_t stream);
int tfe_pdf_replay(const uint32_t* hists, const int64_t* counts, int64_t num_batches, double* pdf,
                   int32_t* iterations, cudaStream_t stream);
int64_t tfe_search_workspace_bytes();
int tfe_search(const aq_tfe_state_t* st, const double* pdf, int stats_updated, const int32_t* stats_updated_dev, int bw,
               int symmetric, int strict, int unsigned_sym, double* out, void* ws, int64_t ws_bytes, cudaStream_t stream);

int tfe_percentile(const aq_tfe_state_t* st, const double* pdf, int stats_updated, const int32_t* stats_updated_dev,
                   float percentile, int bw, int symmetric, int strict, int unsigned_sym, double* out, cudaStream_t stream);
int64_t tfe_mse_workspace_bytes();
int tfe_mse(const aq_tfe_state_t* st, const double* pdf, int stats_updated, const int32_t* stats_updated_dev, int bw,
            int symmetric, int strict, int unsigned_sym, double* out, void* ws, cudaStream_t stream);

int64_t v2hist_scratch_bytes();
int v2hist_collect(const void* x, int dtype, int64_t n, int nb, aq_v2hist_head_t* batch, void* scratch, cudaStream_t st);
int v2hist_merge(const void* x, int dtype, int64_t n, int nb, aq_v2hist_head_t* state, const aq_v2hist_head_t* batch,
                 int state_has_stats, void* scratch, float* updates, cudaStream_t st);
int v2hist_collect_rows(const void* x, int dtype, int64_t n, int rows, int nb, aq_v2hist_head_t* batch,
                        int64_t block_stride, void* scratch, cudaStream_t st);
int v2hist_merge_rows(const void* x, int dtype, int64_t n, int rows, int nb, aq_v2hist_head_t* state,
                      const aq_v2hist_head_t* batch, int64_t block_stride, int state_has_stats, void* scratch,
                      float* updates, cudaStream_t st);
int v2hist_update_rows(const void* x, int dtype, int64_t n, int rows, int nb, aq_v2hist_head_t* state,
                       aq_v2hist_head_t* batch, int64_t block_stride, int state_has_stats, void* scratch,
                       float* updates, cudaStream_t st);
int v2hist_range_rows(const void* x, int dtype, int64_t n, int rows, int32_t* range, void* scratch, cudaStream_t st);
int v2hist_plan_batches(const int32_t* ranges, int n_batches, int rows, int nb, float* plans, cudaStream_t st);
int v2hist_count_rows(const void* x, int dtype, int64_t n, int rows, int nb, const float* plan, uint32_t* counts,
                      cudaStream_t st);
int v2hist_range_many(const void* const* xs, int m, int dtype, int64_t n, int rows, int32_t* ranges, int64_t stride_words,
                      void* scratch, cudaStream_t st);
int v2hist_count_many(const void* const* xs, int m, int dtype, int64_t n, int rows, int nb, const float* plans,
                      int64_t plan_stride, uint32_t* counts, int64_t count_stride, cudaStream_t st);
int v2hist_replay_batches(const uint32_t* counts, const float* plans, int n_batches, int rows, int nb,
                          aq_v2hist_head_t* states, int64_t block_stride, cudaStream_t st);
int v2hist_sqnr_rows(const aq_v2hist_head_t* stats, int64_t block_stride, int rows, int nb, double num_steps,
                     int symmetric, int num_deltas, const float* offsets, int num_offsets, double gamma, float* out,
                     void* ws, int64_t ws_bytes, cudaStream_t st, int out_width = 2, int stats_dtype = 0,
                     double qmin = 0.0);
int64_t v2hist_sqnr_workspace_bytes();
int v2hist_sqnr(const aq_v2hist_head_t* stats, int nb, double num_steps, int symmetric, int num_deltas,
                const float* offsets, int num_offsets, double gamma, float* out, void* ws, int64_t ws_bytes,
                cudaStream_t st);

}   // namespace aq
