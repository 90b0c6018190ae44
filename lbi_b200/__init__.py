"""lbi_b200: Blackwell-native region-parallel training with latent bounded interfaces.

Package layout
--------------
backbones/   Transformer, Mamba-2 (SSD) and Mamba-3 (SISO) blocks and stacks
interfaces/  bounded interface state maps (vector MLP)
canvas/      token-embedding canvas
readouts/    final norm + LM head
backends/    region backends and structured lowerings (input pullback over a basis, parameter VJP)
backward/    autograd, reference-scan and suffix-scan engines
models/      dense and LBI language models, region plans (depth axis and sequence axis)
legacy/      LBI-1 model and checkpoint migration
train/       config, runners, checkpointing, metrics, evaluation
data/        synthetic tasks, byte streams, tokenizers, token shards
ops/         Python entry points of the sm_100a CUDA kernels, each with an fp32 PyTorch oracle
csrc/        CUDA/C++ sources (tcgen05 GEMM, attention pullback, suffix scan, fused elementwise, peer-memory kernels)
parallel/    one-process-per-GPU runtime: symmetric peer buffers, region placement, fused optimizer
utils/       device timing, clocks sampling, NVTX ranges
"""

__version__ = "0.1.0"
