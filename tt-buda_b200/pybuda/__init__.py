"""pybuda: the tensor / data-format conversion surface of TT-Buda, backed by hand-written
sm_100a CUDA kernels (libbuda_cuda.so) behind the reference's backend_api entry points.

Only the data-format path is here: tilize / untilize, Bfp8_b / Bfp4_b / Bfp2_b pack and unpack,
the golden int8 quantise ops and the Bfp8_b-weight matmul.  There is no CPU fallback.
"""
TILE_DIM = 32
