"""Model zoo: Llama (the product model) plus GPT, Gemma, Phi-2, Mamba, RetNet, RoFormer and a
configurable Transformer template."""
