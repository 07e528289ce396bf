// qproj.cuh — what the two projection sources share: the Q8_K image the integer products read.
#pragma once
#include "common.cuh"

// One image per (tile of 8 tokens, super-block of 256 inputs):
//   [0, 2048)     codes: 16 k-steps of 16 inputs x [8 tokens][16 int8]  (word `lane` of a k-step = the int8 MMA
//                 B operand of lane (token lane / 4, inputs 4 (lane % 4) ..))
//   [2048, 2080)  the 8 tokens' scales d (f32)
//   [2080, 2208)  low bytes (unsigned) of the sums of the codes over each run of 32 inputs: [8 tokens][16], 8 used
//   [2208, 2336)  high bytes (signed) of the same sums
constexpr int ORN_Q8K_IMG_D = 2048, ORN_Q8K_IMG_LO = 2080, ORN_Q8K_IMG_HI = 2208, ORN_Q8K_IMG_BYTES = 2336;

size_t orn_q8k_image_bytes(int T, int n_in);
ornith_status orn_q8k_quantize_image(const void *x, int act_dtype, int T, int n_in, void *img, cudaStream_t stream);
