"""B200 (sm_100a) implementation of the fused GPT-NeoX/Pythia decode path of
ClusterFusion++, behind the reference's `clusterfusion` operator API.

    import clusterfusionplus_b200 as clusterfusion
    out, k, v = clusterfusion.pythia_6b9_decoder_layer(...)

Everything computes in libclusterfusion_b200.so (hand-written CUDA); importing
this package fails if that library has not been built.
"""
from ._lib import CF_PYTHIA_2B8, CF_PYTHIA_6B9, CfDims, LIB_PATH  # noqa: F401
from .api import (  # noqa: F401
    device_status, launch_info, llama_decoder_layer, llama_decoder_layer_batch_decode_sglang, llama_decoder_layer_sglang,
    llama_mlp_batch_sglang, llama_mlp_sglang, model_dims,
    pythia_2b8_attention_only, pythia_2b8_create_graph_context, pythia_2b8_decoder_layer,
    pythia_2b8_decoder_layer_split, pythia_2b8_destroy_graph_context, pythia_2b8_graph_decode_step,
    pythia_2b8_graph_set_device_state, pythia_2b8_mlp_only,
    pythia_6b9_create_graph_context, pythia_6b9_decoder_layer, pythia_6b9_decoder_layer_split,
    pythia_6b9_destroy_graph_context, pythia_6b9_graph_decode_step, pythia_6b9_graph_set_device_state,
)
from .checkpoint import convert_state_dict, describe_config, load_decoder  # noqa: F401
from .decoder import PythiaDecoder, rope_table  # noqa: F401
from .llama import LlamaLayerStack  # noqa: F401
from .quality import DecodeQuality, evaluate_decode_quality, step_metrics  # noqa: F401
from .tp import TPDecoder, shard_cache, shard_dims, shard_head_weights, shard_layer_weights  # noqa: F401
