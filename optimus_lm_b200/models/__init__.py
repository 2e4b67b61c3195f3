"""Model zoo: OLMoE, OLMo, Llama, DeepSeek-V3."""
