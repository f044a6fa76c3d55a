"""The `muillm_ext` drop-in exports every function of the reference's torch extension (the m.def list of
csrc/module.cpp:177-432) with the keyword names its Python callers use. Runs without a GPU."""
import inspect

from muillm_b200 import muillm_ext

REFERENCE_FUNCTIONS = """
muillm_linear_forward muillm_parallel_linear_forward muillm_int8_dequantize_forward muillm_int8_linear_forward
muillm_gateupsilu_forward muillm_gateupsilumoe_forward muillm_parallel_gateupsilu_forward
muillm_parallel_gateupsilumoe_forward muillm_gateupsilu_split_forward muillm_parallel_gateupsilu_split_forward
muillm_parallel_gateupsilumoe_split_forward muillm_int8_gateupsilu_dequantize_forward muillm_int8_gateupsilu_forward
muillm_l2norm_forward muillm_qkl2norm_forward muillm_rmsnorm_forward muillm_reduce_sum_forward
muillm_topk_sigmoid_forward muillm_apply_temperature_tuning muillm_add_tokens_check_finished
muillm_rope_forward_no_cache muillm_rope_forward_dynamic_cache muillm_rope_forward_static_cache
muillm_complex_rope_forward_no_cache muillm_static_kvcache_update muillm_sliding_kvcache_update
muillm_causal_transformer_decoding_no_mask muillm_causal_transformer_decoding_masked muillm_engine_init
muillm_sync_init muillm_item_bool muillm_item_f16 muillm_item_f32 muillm_to_cpu muillm_comm_init
muillm_all_reduce_sum muillm_broadcast muillm_linear_module_init muillm_linear_module_deinit
muillm_linear_module_forward muillm_embedding_module_init muillm_embedding_module_deinit
muillm_embedding_module_forward muillm_parallel_linear_module_init muillm_parallel_linear_module_deinit
muillm_parallel_linear_module_forward muillm_parallel_multilinear_module_init
muillm_parallel_multilinear_module_deinit muillm_parallel_multilinear_module_forward
muillm_parallel_gateupdownmlp_module_init muillm_parallel_gateupdownmlp_module_deinit
muillm_parallel_gateupdownmlp_module_forward muillm_parallel_gateupdownmlpmoe_module_init
muillm_parallel_gateupdownmlpmoe_module_deinit muillm_parallel_gateupdownmlpmoe_module_forward
muillm_kvcache_module_get_set_seen_tokens muillm_static_kvcache_module_init muillm_static_kvcache_module_deinit
muillm_static_kvcache_module_sync_back muillm_dynamic_kvcache_module_init muillm_dynamic_kvcache_module_deinit
muillm_dynamic_kvcache_module_sync_back muillm_hybrid_chunked_kvcache_module_init
muillm_hybrid_chunked_kvcache_module_update muillm_hybrid_chunked_kvcache_module_deinit
muillm_hybrid_chunked_kvcache_module_sync_back muillm_rotary_embedding_module_init
muillm_rotary_embedding_module_deinit muillm_rotary_embedding_module_forward muillm_parallel_attention_module_init
muillm_parallel_attention_module_deinit muillm_parallel_attention_module_forward
muillm_parallel_attention_module_rope_forward muillm_parallel_llama4_attention_module_init
muillm_parallel_llama4_attention_module_deinit muillm_parallel_llama4_attention_module_forward
muillm_parallel_llama4_attention_module_rope_forward muillm_parallel_decoder_module_init
muillm_parallel_decoder_module_deinit muillm_parallel_decoder_module_forward
muillm_parallel_llama4_decoder_module_init muillm_parallel_llama4_decoder_module_deinit
muillm_parallel_llama4_decoder_module_forward muillm_parallel_decoder_stack_init
muillm_parallel_decoder_stack_deinit muillm_parallel_decoder_stack_forward
muillm_parallel_llama4_decoder_stack_init muillm_parallel_llama4_decoder_stack_deinit
muillm_parallel_llama4_decoder_stack_forward
""".split()

# keyword names the reference declares with py::arg (its Python calls some of these by keyword)
KEYWORDS = {
    "muillm_linear_forward": ["engine", "x", "weights", "norm_weights", "epsilon", "mul_bias", "add_bias", "residual"],
    "muillm_parallel_linear_forward": ["engine", "comm", "x", "weights", "norm_weights", "epsilon", "mul_bias",
                                       "add_bias", "residual", "sharding_dim", "reduce"],
    "muillm_parallel_gateupsilu_forward": ["engine", "comm", "norm_weights", "epsilon", "gate_weights", "up_weights",
                                           "down_weights", "residual", "x", "reduce"],
    "muillm_parallel_gateupsilumoe_forward": ["engine", "comm", "num_shared_experts", "num_dynamic_experts",
                                              "norm_weights", "epsilon", "gate_weights", "up_weights", "down_weights",
                                              "residual", "x", "router_scores", "router_indices", "reduce"],
    "muillm_apply_temperature_tuning": ["query_states", "cache_position", "attn_scale", "floor_scale"],
    "muillm_add_tokens_check_finished": ["input_ids", "next_tokens", "unfinished_sequences",
                                         "has_eos_stopping_criteria", "pad_token_id", "eos_token_id",
                                         "has_max_length_stopping_criteria", "max_length"],
    "muillm_linear_module_init": ["engine", "weights", "norm_weights", "epsilon", "mul_bias", "add_bias"],
    "muillm_linear_module_forward": ["module", "inputs", "residual"],
    "muillm_embedding_module_init": ["engine", "weights"],
    "muillm_parallel_linear_module_init": ["engine", "comm", "weights", "norm_weights", "epsilon", "mul_bias",
                                           "add_bias", "sharding_dim"],
    "muillm_parallel_linear_module_forward": ["module", "inputs", "residual", "reduce"],
    "muillm_parallel_multilinear_module_init": ["engine", "comm", "linear", "slices", "sharding_dim"],
    "muillm_parallel_multilinear_module_forward": ["module", "input", "collect_outputs"],
    "muillm_parallel_gateupdownmlp_module_init": ["engine", "comm", "method", "norm_weights", "gate_weights",
                                                  "up_weights", "down_weights", "variance_epsilon"],
    "muillm_parallel_gateupdownmlp_module_forward": ["module", "inputs", "residual", "reduce"],
    "muillm_parallel_gateupdownmlpmoe_module_init": ["engine", "comm", "router", "num_shared_experts",
                                                     "num_dynamic_experts", "num_routed_experts", "norm_weights",
                                                     "gate_weights", "up_weights", "down_weights", "variance_epsilon"],
    "muillm_kvcache_module_get_set_seen_tokens": ["module", "seen_tokens"],
    "muillm_static_kvcache_module_init": ["engine", "key_cache", "value_cache", "seen_tokens"],
    "muillm_hybrid_chunked_kvcache_module_init": ["engine", "key_cache", "value_cache", "is_sliding", "window_size",
                                                  "seen_tokens"],
    "muillm_hybrid_chunked_kvcache_module_update": ["module", "key_states", "value_states", "cache_position",
                                                    "layer_index"],
    "muillm_rotary_embedding_module_init": ["engine", "layer_idx", "cos_cached", "sin_cached"],
    "muillm_rotary_embedding_module_forward": ["module", "cache", "q_in", "k_in", "v_in", "position_ids", "cos_sin",
                                               "cache_positions"],
    "muillm_parallel_attention_module_init": ["engine", "comm", "rotary", "o_proj", "num_tp_heads",
                                              "num_tp_key_value_heads", "head_dim"],
    "muillm_parallel_attention_module_forward": ["module", "q", "k", "v", "m", "residual"],
    "muillm_parallel_attention_module_rope_forward": ["module", "cache", "q", "k", "v", "m", "residual", "position_ids",
                                                      "cos_sin", "cache_positions"],
    "muillm_parallel_llama4_attention_module_init": ["engine", "comm", "o_proj", "num_tp_heads",
                                                     "num_tp_key_value_heads", "head_dim", "use_rope", "use_qk_norm",
                                                     "norm_epsilon", "use_temperature_tuning", "attention_scale",
                                                     "floor_scale", "layer_index"],
    "muillm_parallel_llama4_attention_module_rope_forward": ["module", "cache", "q", "k", "v", "m", "residual",
                                                             "position_embeds", "cache_positions"],
    "muillm_parallel_decoder_module_init": ["engine", "comm", "multilinear", "attention", "mlp"],
    "muillm_parallel_decoder_module_forward": ["module", "cache", "h", "m", "position_ids", "cos_sin",
                                               "cache_positions"],
    "muillm_parallel_llama4_decoder_module_init": ["engine", "comm", "multilinear", "attention", "mlp",
                                                   "use_chunked_attention"],
    "muillm_parallel_llama4_decoder_module_forward": ["module", "cache", "h", "mask", "chunked_mask", "position_embeds",
                                                      "cache_positions"],
    "muillm_parallel_decoder_stack_init": ["engine", "comm", "embed_tokens_module", "rotary_emb_module", "decoders"],
    "muillm_parallel_decoder_stack_forward": ["module", "cache", "input_ids", "input_embeds", "m", "position_ids",
                                              "cache_positions"],
    "muillm_parallel_llama4_decoder_stack_init": ["engine", "comm", "decoders"],
    "muillm_parallel_llama4_decoder_stack_forward": ["module", "cache", "h", "mask", "chunked_mask", "position_embeds",
                                                     "cache_positions"],
}


def test_every_reference_function_is_exported():
    assert len(REFERENCE_FUNCTIONS) == 89 and len(set(REFERENCE_FUNCTIONS)) == 89
    missing = [n for n in REFERENCE_FUNCTIONS if not callable(getattr(muillm_ext, n, None))]
    assert not missing, f"missing from the drop-in: {missing}"


def test_keyword_names_match_the_reference():
    for name, want in KEYWORDS.items():
        got = [p for p in inspect.signature(getattr(muillm_ext, name)).parameters if p != "flags"]
        assert got == want, f"{name}: {got} != {want}"


def test_defaults_of_the_reference():
    sig = inspect.signature(muillm_ext.muillm_parallel_linear_forward)
    assert sig.parameters["sharding_dim"].default == 1 and sig.parameters["reduce"].default is False
    assert inspect.signature(muillm_ext.muillm_parallel_linear_module_forward).parameters["reduce"].default is False
    assert inspect.signature(muillm_ext.muillm_parallel_gateupdownmlp_module_forward).parameters["reduce"].default is True
    assert inspect.signature(muillm_ext.muillm_parallel_gateupsilu_forward).parameters["reduce"].default is True


def test_handles_are_default_constructible_classes_and_world_one_needs_no_peers():
    assert isinstance(muillm_ext.muillm_engine_ptr(), muillm_ext.muillm_engine_ptr)
    assert isinstance(muillm_ext.muillm_synchronizer_ptr(), muillm_ext.muillm_synchronizer_ptr)
    comm = muillm_ext.muillm_comm_init(None, 1, 1, 0, 0)
    assert isinstance(comm, muillm_ext.muillm_comm_ptr) and comm.comm is None


def test_seen_tokens_only_moves_forward():
    c = muillm_ext.muillm_static_kvcache_module_init(None, [], [], 5)
    assert muillm_ext.muillm_kvcache_module_get_set_seen_tokens(c, 3) == 5
    assert muillm_ext.muillm_kvcache_module_get_set_seen_tokens(c, 9) == 9
