"""transformers_fusion_b200 — a Blackwell (B200, sm_100a) native LLM training, quantization and
serving framework: PyTorch for the tensor/autograd layer, hand-written tcgen05/TMA CUDA kernels for
the hot ops, fused compute+collective kernels over NVLink peer memory, C++ for the codec, tokenizer
and HTTP server."""
__version__ = "0.1.0"
