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
cuda/        the kernel entry points under the reference's module paths (cuda.interface, cuda.transformer, cuda.mamba3)
scripts/     paper launchers and presets, post-hoc evaluation, figures, gradient-parity report
benchmarks/  microbenchmarks (GEMM, attention, SSD, communication paths) and small profiling cases
utils/       failure handling (heartbeats, watchdog, host-side fault injection), NVTX ranges, gradient-parity harness
inference.py token-by-token decoding (bounded memory for sequence-axis models), generate(), generation command
serve.py     HTTP front end for generation (FastAPI / uvicorn when installed)
"""

__version__ = "0.2.0"
