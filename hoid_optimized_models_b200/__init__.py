"""B200-native (sm_100a) kernels and engines for the hot path of hoid-optimized-models.

    ops          torch custom ops `b200::<op>` over the C ABI of include/b200ops.h
    decoder      Llama-3.1 / Qwen3 / Qwen3-MoE engines (tensor- and expert-parallel)
    encoder      XLM-RoBERTa engine (data-parallel)
    whisper      Whisper encoder and cached decoder
    checkpoint   HuggingFace safetensors checkpoints under the names the engines read
    weights      seeded synthetic checkpoints, RoPE tables
    configs      model shapes and the algorithmic bytes per decoded token
    tp, comm     weight sharding; peer-memory link of the fused all-reduce
    build        nvcc -> libb200ops.so (in-tree)

Importing the package does not load the library; the first op call does, and fails loudly if the
library has not been built - there is no CPU path.
"""
