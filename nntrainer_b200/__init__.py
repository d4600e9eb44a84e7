"""nntrainer_b200: NNTrainer's block-quantized weight matmul path (Q4_0 / Q4_K /
Q6_K weights x Q8_0 / Q8_K activations) as hand-written CUDA kernels for
sm_100a, behind a C ABI (include/nntr_cuda.h). ``backend`` mirrors the names of
the reference's cpu_backend functions for that path."""
from . import capi  # noqa: F401
