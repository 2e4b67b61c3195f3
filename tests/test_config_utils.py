import pytest

from optimus_lm_b200 import config_utils as cu
from optimus_lm_b200.models.olmoe.configuration_olmoe import OlmoeParallelConfig
from optimus_lm_b200.models.deepseek_v3.configuration_deepseek_v3 import DeepseekV3ParallelConfig


def test_olmoe_tags():
    c = cu.get_modified_config("allenai/OLMoE-1B-7B-0924--SA3-SH1.5-SE2.25-SC0.5-SI2-L36", OlmoeParallelConfig())
    assert (c.num_hidden_layers, c.num_attention_heads, c.hidden_size) == (36, 48, 3072)
    assert (c.num_experts, c.num_experts_per_tok, c.intermediate_size) == (144, 4, 2048)
    assert c.output_router_logits is True and c.skip_qk_norm is False
    c = cu.get_modified_config("allenai/OLMoE-1B-7B-0924--SM1.5-SE1.125-NAL", OlmoeParallelConfig())
    assert (c.num_attention_heads, c.hidden_size, c.num_experts) == (24, 3072, 72)
    assert c.output_router_logits is False
    c = cu.get_modified_config("allenai/OLMoE-1B-7B-0924--S2-SKIPQKNORM", OlmoeParallelConfig())
    assert (c.num_attention_heads, c.hidden_size, c.num_experts, c.intermediate_size) == (32, 4096, 128, 2048)
    assert c.skip_qk_norm is True
    with pytest.raises(AssertionError):
        cu.get_modified_config("allenai/OLMoE-1B-7B-0924--S2-SA2", OlmoeParallelConfig())
    with pytest.raises(AssertionError):
        cu.get_modified_config("allenai/OLMoE-1B-7B-0924--XX2", OlmoeParallelConfig())


def test_dsv3_tags():
    c = cu.get_modified_config("deepseek-ai/DeepSeek-V3--L4-DL1-N264-K4-MI1024-A64-SE2-H4096-I8192",
                               DeepseekV3ParallelConfig())
    assert (c.num_hidden_layers, c.first_k_dense_replace, c.n_routed_experts, c.num_experts_per_tok) == (4, 1, 264, 4)
    assert (c.moe_intermediate_size, c.num_attention_heads, c.num_key_value_heads) == (1024, 64, 64)
    assert (c.n_shared_experts, c.hidden_size, c.intermediate_size) == (2, 4096, 8192)


def test_olmo_llama_offline_build():
    c = cu.build_config("allenai/OLMo-1B-hf--L4-RMS-TWE", tensor_parallelism=2)
    assert c.num_hidden_layers == 4 and c.use_rms_norm and c.tie_word_embeddings
    assert c.max_position_embeddings == 4096 and c.tensor_parallelism == 2
    c = cu.build_config("meta-llama/Llama-3.1-8B--L2-H1024-I2048")
    assert (c.num_hidden_layers, c.hidden_size, c.intermediate_size, c.head_dim) == (2, 1024, 2048, 32)


def test_cached_model_key():
    k = cu.cached_model_key("allenai/OLMoE-1B-7B-0924--L4-NAL", 2, 4, 1, 1, merged_mlp=True)
    assert k == "allenai__OLMoE-1B-7B-0924--L4_pp2-ep4-tp1-vpp1_mmlp"
    k = cu.cached_model_key("allenai/OLMoE-1B-7B-0924--NAL", 1, 1, 1, 1)
    assert k == "allenai__OLMoE-1B-7B-0924_pp1-ep1-tp1-vpp1"
