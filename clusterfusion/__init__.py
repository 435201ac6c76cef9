"""Drop-in name of the reference package: `import clusterfusion` keeps working
(clusterfusion/__init__.py:6-16 of the reference re-exports its native module the
same way)."""
from clusterfusionplus_b200 import *  # noqa: F401,F403
from clusterfusionplus_b200 import (  # noqa: F401
    llama_decoder_layer, llama_decoder_layer_batch_decode_sglang, llama_decoder_layer_sglang,
    pythia_2b8_attention_only, pythia_2b8_create_graph_context, pythia_2b8_decoder_layer,
    pythia_2b8_decoder_layer_split, pythia_2b8_destroy_graph_context, pythia_2b8_graph_decode_step,
    pythia_2b8_mlp_only, pythia_6b9_create_graph_context, pythia_6b9_decoder_layer,
    pythia_6b9_destroy_graph_context, pythia_6b9_graph_decode_step,
)
