// Runs the reference's kernels (compiled as host C++ by oracle/build_ref.py) block by block on CPU
// threads and exports one C function per kernel.  TEST INFRASTRUCTURE ONLY: nothing in the product
// links or loads this.  Signatures follow the reference's templates:
//   kv_cache_append.hip.template:13-22, flash_attention_split_kv_partial.hip.template:31-45,
//   flash_attention_split_kv_reduce.hip.template:14-22, flash_attention.hip.template:29-43,
//   rope.hip.template:17-35.
#include <hip/hip_runtime.h>
#include <hip/hip_fp16.h>
#include <pthread.h>
#include <functional>
#include <thread>
#include <vector>

thread_local dim3 threadIdx;
dim3 blockIdx, blockDim, gridDim;
float smem[1 << 16];

static pthread_barrier_t g_barrier;
void vte_ref_block_barrier() { pthread_barrier_wait(&g_barrier); }

extern "C" {
void kv_cache_append_kernel(const __half*, const __half*, __half*, __half*, int, int, const int*, int);
void flash_attention_split_kv_partial_kernel(const __half*, const __half*, const __half*, float*, float*, float*, int, int,
                                             int, float, const int*, int, int);
void flash_attention_split_kv_reduce_kernel(const float*, const float*, const float*, __half*, int, int, int);
void flash_attention_kernel(const __half*, const __half*, const __half*, __half*, __half*, __half*, int, int, int, int, float,
                            const int*, int);
void rope_kernel(__half*, __half*, const __half*, const __half*, int, int, int, int, const int*, int, int);
}

// grid (gx, gy, gz), block (bx, 1, 1): every block in turn, its threads as std::threads that meet at
// __syncthreads.  A thread that returns early must not leave the others waiting: the reference's
// kernels only return early for a whole block at once or before the first barrier with
// blockDim.x == head_dim, which is how they are launched here.
static void launch(unsigned gx, unsigned gy, unsigned gz, unsigned bx, const std::function<void()>& body) {
    gridDim = {gx, gy, gz};
    blockDim = {bx, 1, 1};
    for (unsigned z = 0; z < gz; ++z)
        for (unsigned y = 0; y < gy; ++y)
            for (unsigned x = 0; x < gx; ++x) {
                blockIdx = {x, y, z};
                pthread_barrier_init(&g_barrier, nullptr, bx);
                std::vector<std::thread> threads;
                threads.reserve(bx);
                for (unsigned t = 0; t < bx; ++t)
                    threads.emplace_back([t, &body] {
                        threadIdx = {t, 0, 0};
                        body();
                    });
                for (auto& th : threads) th.join();
                pthread_barrier_destroy(&g_barrier);
            }
}

extern "C" {

void vte_ref_kv_cache_append(const void* k, const void* v, void* k_cache, void* v_cache, int batch, int num_kv_heads,
                             int head_dim, const int* kv_offsets, int kv_batch_stride) {
    launch(batch, num_kv_heads, 1, head_dim, [&] {
        kv_cache_append_kernel((const __half*)k, (const __half*)v, (__half*)k_cache, (__half*)v_cache, num_kv_heads, head_dim,
                               kv_offsets, kv_batch_stride);
    });
}

void vte_ref_split_kv_partial(const void* q, const void* k_cache, const void* v_cache, float* partial_m, float* partial_l,
                              float* partial_o, int batch, int num_q_heads, int num_kv_heads, int head_dim, float scale,
                              const int* kv_offsets, int kv_batch_stride, int max_chunks) {
    launch(batch, num_q_heads, max_chunks, head_dim, [&] {
        flash_attention_split_kv_partial_kernel((const __half*)q, (const __half*)k_cache, (const __half*)v_cache, partial_m,
                                                partial_l, partial_o, num_q_heads, num_kv_heads, head_dim, scale, kv_offsets,
                                                kv_batch_stride, max_chunks);
    });
}

void vte_ref_split_kv_reduce(const float* partial_m, const float* partial_l, const float* partial_o, void* output, int batch,
                             int num_q_heads, int head_dim, int max_chunks) {
    launch(batch, num_q_heads, 1, head_dim, [&] {
        flash_attention_split_kv_reduce_kernel(partial_m, partial_l, partial_o, (__half*)output, num_q_heads, head_dim, max_chunks);
    });
}

void vte_ref_flash_attention(const void* q, const void* k, const void* v, void* k_cache, void* v_cache, void* output, int batch,
                             int seq_len, int num_q_heads, int num_kv_heads, int head_dim, float scale, const int* kv_offsets,
                             int kv_batch_stride) {
    launch(batch, num_q_heads, 1, head_dim, [&] {
        flash_attention_kernel((const __half*)q, (const __half*)k, (const __half*)v, (__half*)k_cache, (__half*)v_cache,
                               (__half*)output, seq_len, num_q_heads, num_kv_heads, head_dim, scale, kv_offsets, kv_batch_stride);
    });
}

void vte_ref_rope(void* q, void* k, const void* cos_cache, const void* sin_cache, int grid_x, int grid_y, int block_x, int seq_len,
                  int num_q_heads, int num_kv_heads, int head_dim, const int* kv_offsets, int rope_type, int rotary_dim) {
    launch(grid_x, grid_y, 1, block_x, [&] {
        rope_kernel((__half*)q, (__half*)k, (const __half*)cos_cache, (const __half*)sin_cache, seq_len, num_q_heads, num_kv_heads,
                    head_dim, kv_offsets, rope_type, rotary_dim);
    });
}

int vte_ref_split_kv_chunk_size() { return VTE_REF_SPLIT_KV_CHUNK_SIZE; }

}  // extern "C"
