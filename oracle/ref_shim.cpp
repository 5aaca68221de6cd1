// Host-side shim that compiles the reference's scorer kernel text, unmodified, as C++.
// TEST INFRASTRUCTURE ONLY.
//
// The reference kernel (GPT-FAST/kernels/soft_hash_collision.cu:25-54 in the reference
// tree) is plain scalar code that only touches blockIdx / threadIdx / blockDim, so it can
// be executed on the CPU by defining those names and looping over the launch grid its own
// header comment documents (block 256, grid (ceil(T/256), H, B)).  The kernel source is
// NOT copied here: the build recipe passes its path as SOCKET_REF_KERNEL_SRC and the
// preprocessor includes it where it lies.
#include <cmath>
#include <cstdint>

#define __global__
#define __restrict__

namespace {
struct Dim3 { int x, y, z; };
thread_local Dim3 blockIdx{0, 0, 0};
thread_local Dim3 threadIdx{0, 0, 0};
thread_local Dim3 blockDim{256, 1, 1};
}  // namespace

#include SOCKET_REF_KERNEL_SRC

extern "C" void ref_soft_hash_collision(const float* q_probs, const int16_t* key_buckets,
                                        const bool* allowed, const float* v_hist, float* out,
                                        int B, int H, int L, int R, int T_k) {
    const int threads = 256;
    const int nblk = (T_k + threads - 1) / threads;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b) {
        for (int h = 0; h < H; ++h) {
            for (int bx = 0; bx < nblk; ++bx) {
                for (int tx = 0; tx < threads; ++tx) {
                    blockIdx = Dim3{bx, h, b};
                    threadIdx = Dim3{tx, 0, 0};
                    blockDim = Dim3{threads, 1, 1};
                    soft_hash_collision_kernel_3(q_probs, key_buckets, allowed, v_hist, out,
                                                 B, H, L, R, T_k);
                }
            }
        }
    }
}
