// TEST INFRASTRUCTURE ONLY -- never linked into the shipped library.
//
// C entry point around the reference's own nearest-neighbour extension, compiled by the Makefile beside this
// file with nvcc from where the source lies (macro REF_KNN_CU = submodules/simple-knn/simple_knn.cu; its torch
// binding, ext.cpp / spatial.cu, is three lines around SimpleKNN::knn and is replaced by this function).
// Device code: it runs on the GPU box only, to generate tests/golden/knn.npz (tests/golden/make_knn_golden.py).
#include REF_KNN_CU

// points [n,3] and mean_dist2 [n] are device pointers; synchronises before it returns.
extern "C" int ref_knn_mean_dist2(int n, float* points, float* mean_dist2) {
    SimpleKNN::knn(n, reinterpret_cast<float3*>(points), mean_dist2);
    cudaError_t e = cudaDeviceSynchronize();
    return e == cudaSuccess ? 0 : (int)e;
}
