// Internal launch interface between the C ABI (plx_abi.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace plx {

struct TrainArgs;
struct DecodeArgs;
struct ExchangeArgs;

// Every kernel launch of this library goes through count_launch() so that
// plx_kernel_launch_count() can report how many ran.
void count_launch();

int launch_train_fwd_mma(const TrainArgs &a, int dtype, int head_dim, cudaStream_t stream);
int launch_train_bwd_mma(const TrainArgs &a, int dtype, int head_dim, int stages, cudaStream_t stream);

// tcgen05 + TMEM + TMA forward (head_dim 128, no sliding window); `supported` decides per problem
bool train_fwd_sm100_supported(const TrainArgs &a, int head_dim);
int launch_train_fwd_sm100(const TrainArgs &a, int dtype, int head_dim, cudaStream_t stream);
// Error words of the current device (see sm100::ErrSink): `word` in device memory, `mirror` in mapped
// pinned host memory.  Both null on failure.  The first call on a device allocates the mirror.
struct ErrorWords {
    int *word, *mirror;
};
ErrorWords sm100_error_words();
int sm100_error_word(int *value, bool clear);   // synchronises the device
int sm100_error_peek(int *value, bool clear);   // reads (and optionally clears) the host mirror only: no synchronisation
// tcgen05 backward: stage is PLX_BWD_DQR or PLX_BWD_DKV (the row statistics must already be in a.bst)
bool train_bwd_sm100_supported(const TrainArgs &a, int head_dim);
int launch_train_bwd_sm100(const TrainArgs &a, int dtype, int head_dim, int stage, cudaStream_t stream);

constexpr int kDecodeGqaWarps = 8;   // warps (independent splits) per CTA of the grouped-query decode kernel
int launch_decode(const DecodeArgs &a, int dtype, int head_dim, cudaStream_t stream);
bool decode_fused_exchange_supported(const DecodeArgs &a);   // see exchange_merge_warp in plx_decode.cu
int launch_decode_exchange_merge(const ExchangeArgs &x, const float *part, int head_dim, int dtype, void *out,
                                 const ErrorWords &err, cudaStream_t stream);
int launch_decode_merge(const float *parts, int n_parts, int n_records, int head_dim, int dtype, void *out,
                        cudaStream_t stream);

}  // namespace plx
