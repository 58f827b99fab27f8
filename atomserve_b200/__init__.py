"""atomserve_b200: a small, whole LLM inference engine for one B200.

Token ids in, token ids out, for the Qwen3 dense architecture: typed configuration and an
architecture registry (`config`), safetensors loading and seeded random models (`weights`),
layers assembled from interchangeable parts (`parts`, `models`), a paged cache manager with
per-request state slots (`cache`), one step function with a continuous-batching scheduler
above it (`engine`), sampling (`sampling`), and hand-written CUDA kernels for sm_100a
(`csrc`, wrapped by `ops`).
"""

__version__ = "0.1.0"
