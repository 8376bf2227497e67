// Internal launch interface between the C ABI (plx_abi.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace plx {

struct TrainArgs;
struct DecodeArgs;

// Every kernel launch of this library goes through count_launch() so that
// plx_kernel_launch_count() can report how many ran.
void count_launch();

int launch_train_fwd_mma(const TrainArgs &a, int dtype, int head_dim, cudaStream_t stream);
int launch_train_bwd_mma(const TrainArgs &a, int dtype, int head_dim, int stages, cudaStream_t stream);

int launch_decode(const DecodeArgs &a, int dtype, int head_dim, cudaStream_t stream);
int launch_decode_merge(const float *parts, int n_parts, int n_records, int head_dim, int dtype, void *out,
                        cudaStream_t stream);

}  // namespace plx
