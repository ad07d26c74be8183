"""DeepBench problem sets (Baidu DeepBench, as tabulated in deep500 samples/deepbench/deepbench.py): GEMM sizes
(M, N, K, transpose A, transpose B) and convolution sizes (W, H, C, N, K, S, R, pad_w, pad_h, stride_w, stride_h).
A subset that fits the tensor-core kernels' alignment rules, plus the ResNet-50 shapes."""

GEMM = [(1760, 16, 1760, False, False), (1760, 128, 1760, False, False), (1760, 7000, 1760, False, False),
        (2048, 64, 2048, False, False), (2048, 7000, 2048, False, False), (2560, 128, 2560, False, False),
        (4096, 128, 4096, False, False), (4096, 7000, 4096, False, False), (5124, 9124, 1760, False, False),
        (3072, 128, 1024, False, False), (7680, 5481, 2560, False, False), (512, 24000, 1530, False, False),
        (1024, 16, 512, True, False), (2048, 128, 2048, True, False), (4096, 7000, 4096, True, False),
        (1760, 7133, 1760, False, True), (4096, 7133, 4096, False, True)]

CONV = [(112, 112, 64, 8, 128, 3, 3, 1, 1, 1, 1), (56, 56, 128, 8, 256, 3, 3, 1, 1, 1, 1),
        (28, 28, 256, 8, 512, 3, 3, 1, 1, 1, 1), (14, 14, 512, 8, 512, 3, 3, 1, 1, 1, 1),
        (7, 7, 512, 8, 512, 3, 3, 1, 1, 1, 1), (56, 56, 64, 16, 64, 3, 3, 1, 1, 1, 1),
        (56, 56, 64, 16, 256, 1, 1, 0, 0, 1, 1), (28, 28, 128, 16, 128, 3, 3, 1, 1, 1, 1),
        (28, 28, 512, 16, 128, 1, 1, 0, 0, 1, 1), (14, 14, 256, 16, 256, 3, 3, 1, 1, 1, 1),
        (14, 14, 1024, 16, 256, 1, 1, 0, 0, 1, 1), (7, 7, 512, 16, 512, 3, 3, 1, 1, 1, 1),
        (7, 7, 2048, 16, 512, 1, 1, 0, 0, 1, 1)]
