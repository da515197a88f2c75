"""The kernel modules that the tests need beyond the package's defaults: attention at the tiny
configurations' head sizes and at those of the reference's op tests, and the test build of the tensor-core product.  A build step may compile them ahead of the tests; a test that meets
a module that is not built compiles it itself at first use."""

TEST_MODULES = [
    *[("attention_simt.cu", {"LLB_HEAD_DIM": d}) for d in (4, 8, 10, 16, 20, 24, 32, 48, 80, 160)],
    *[("attention_mma.cu", {"LLB_HEAD_DIM": d}) for d in (16, 32, 48, 80)],
    # the build in which a bounded wait can be made to run out (test_gpu_kernels.py)
    ("gemm_tc.cu", {"LLB_WAIT_LIMIT": 4096, "LLB_TEST_STALL": 1}),
]
