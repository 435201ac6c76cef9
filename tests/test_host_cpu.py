"""Host-side checks that need no GPU: the C ABI exports what the header declares,
the Python operator surface mirrors the reference's, argument validation, and the
static work split the kernel uses."""
import ctypes
import inspect
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "clusterfusion_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cf_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from clusterfusionplus_b200 import _lib
    syms = header_symbols()
    assert len(syms) >= 20
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in syms:
        assert hasattr(raw, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == syms


def test_header_is_plain_c_and_links_against_the_library(tmp_path):
    """The boundary is a C ABI: the header compiles as C99 and as C++11 without torch or CUDA headers,
    and a C program linked against the shared library resolves and calls an entry point."""
    import shutil
    import subprocess
    from clusterfusionplus_b200 import _lib
    if not shutil.which("gcc") or not shutil.which("g++"):
        pytest.skip("no host compiler")
    src = tmp_path / "use_header.c"
    src.write_text('#include <stdio.h>\n#include "clusterfusion_b200.h"\n'
                   'int main(void) { CfDims d; int rc = cf_model_dims(CF_PYTHIA_6B9, &d);\n'
                   '  printf("%d %d %d %d\\n", rc, d.hidden, d.heads, d.head_dim); return rc; }\n')
    inc = os.path.join(ROOT, "include")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", "-I", inc, str(src)], check=True)
    subprocess.run(["g++", "-std=c++11", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++", "-I", inc, str(src)], check=True)
    exe = tmp_path / "use_header"
    libdir = os.path.dirname(_lib.LIB_PATH)
    subprocess.run(["gcc", "-std=c99", "-I", inc, str(src), "-o", str(exe), "-L", libdir, "-lclusterfusion_b200",
                    f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert out == ["0", "4096", "32", "128"]


def test_error_string_without_gpu():
    """No CPU fallback: on a box without a CUDA device the entry points fail and say why."""
    from clusterfusionplus_b200 import _lib
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    d = _lib.CfDims()
    assert _lib.lib.cf_model_dims(1, ctypes.byref(d)) == 0 and d.hidden == 4096 and d.head_dim == 128
    assert _lib.lib.cf_model_dims(7, ctypes.byref(d)) != 0
    assert "unknown model" in _lib.last_error()
    s = ctypes.c_int(0)
    assert _lib.lib.cf_get_status(ctypes.byref(s)) != 0
    assert _lib.last_error() != ""


REFERENCE_SURFACE = [
    # names of include/pybind.cpp:285-297 of the reference, with their arity
    ("pythia_2b8_decoder_layer", 18), ("pythia_2b8_decoder_layer_split", 18), ("pythia_2b8_attention_only", 16),
    ("pythia_2b8_mlp_only", 5), ("pythia_2b8_create_graph_context", 8), ("pythia_2b8_graph_decode_step", 15),
    ("pythia_2b8_destroy_graph_context", 1), ("pythia_6b9_decoder_layer", 18), ("pythia_6b9_create_graph_context", 8),
    ("pythia_6b9_graph_decode_step", 15), ("pythia_6b9_destroy_graph_context", 1),
]


def test_drop_in_module_surface():
    import clusterfusion
    for name, _ in REFERENCE_SURFACE:
        assert callable(getattr(clusterfusion, name)), name
    sig = inspect.signature(clusterfusion.pythia_2b8_attention_only)
    assert len(sig.parameters) == 16
    assert len(inspect.signature(clusterfusion.pythia_2b8_mlp_only).parameters) == 5


def test_transposed_llama_entry_point_is_a_documented_refusal():
    """The reference's llama_decoder_layer (include/pybind.cpp:66-74) takes transposed weights; the name
    exists and says which entry point computes the same block."""
    import clusterfusion
    assert len(inspect.signature(clusterfusion.llama_decoder_layer).parameters) == 8
    with pytest.raises(NotImplementedError, match="llama_decoder_layer_sglang"):
        clusterfusion.llama_decoder_layer(*[None] * 8)


def test_batch_recording_state_machine_without_gpu():
    """cf_batch_begin / cf_batch_end / cf_batch_abort: misuse is reported, an empty batch is a no-op."""
    from clusterfusionplus_b200 import _lib
    lib = _lib.lib
    assert lib.cf_batch_end(None) != 0 and "cf_batch_begin" in _lib.last_error()
    assert lib.cf_batch_begin() == 0
    assert lib.cf_batch_begin() != 0 and "already open" in _lib.last_error()
    assert lib.cf_batch_abort() == 0
    assert lib.cf_batch_begin() == 0
    assert lib.cf_batch_end(None) == 0          # nothing recorded: nothing to launch, no device needed
    assert lib.cf_batch_end(None) != 0


def test_cpu_tensors_are_rejected():
    import clusterfusion
    H, F = 2560, 10240
    z = lambda *s: torch.zeros(*s, dtype=torch.float16)
    args = [z(1, H), z(3 * H, H), z(3 * H), z(H, H), z(H), z(8, H), z(8, H), z(H), z(H),
            torch.zeros(20), torch.zeros(20), z(H), z(H), z(F, H), z(F), z(H, F), z(H), 3]
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        clusterfusion.pythia_2b8_decoder_layer(*args)


def test_new_entry_points_validate_before_touching_the_device():
    """Argument errors of the prefill GEMM and the Llama MLP block are reported with a message,
    GPU or not; with good arguments and no GPU the call fails on the missing device."""
    from clusterfusionplus_b200 import _lib
    lib = _lib.lib
    one = ctypes.c_void_p(16)  # never dereferenced: validation comes first
    assert lib.cf_prefill_linear(one, one, None, None, one, 4, 1020, 1024, 0, None) != 0
    assert "multiples of 8" in _lib.last_error()
    assert lib.cf_prefill_linear(one, one, None, one, one, 4, 1024, 1024, _lib.CF_ACT_GELU_TANH, None) != 0
    assert "residual" in _lib.last_error()
    assert lib.cf_prefill_linear(one, one, None, None, one, 4, 1024, 1024, 9, None) != 0
    assert "activation" in _lib.last_error()
    assert lib.cf_prefill_linear(None, one, None, None, one, 4, 1024, 1024, 0, None) != 0
    assert lib.cf_llama_mlp_sglang(one, None, one, one, one, 1e-5, 11007, one, one, None) != 0
    assert "ffn" in _lib.last_error()
    assert lib.cf_llama_mlp_sglang(one, one, one, one, one, 1e-5, 11008, one, one, None) != 0
    assert "alias" in _lib.last_error()
    if not torch.cuda.is_available():
        assert lib.cf_prefill_linear(one, one, None, None, one, 4, 1024, 1024, 0, None) != 0
        assert _lib.last_error() != ""


def test_checkpoint_adaptor_edge_cases():
    """Tied LM head, missing attention biases and a wrong tensor shape."""
    import clusterfusionplus_b200 as cf
    from transformers import GPTNeoXConfig
    cfg = GPTNeoXConfig(hidden_size=256, num_attention_heads=2, intermediate_size=512, num_hidden_layers=1,
                        vocab_size=64, rotary_pct=0.25, hidden_act="gelu_new")
    d, flags, base = cf.describe_config(cfg)
    assert (d.head_dim, d.rotary, flags) == (128, 32, 0)
    H, F, V = 256, 512, 64
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)
    sd = {"gpt_neox.embed_in.weight": r(V, H), "gpt_neox.final_layer_norm.weight": r(H), "gpt_neox.final_layer_norm.bias": r(H)}
    pre = "gpt_neox.layers.0."
    sd.update({pre + "input_layernorm.weight": r(H), pre + "input_layernorm.bias": r(H),
               pre + "post_attention_layernorm.weight": r(H), pre + "post_attention_layernorm.bias": r(H),
               pre + "attention.query_key_value.weight": r(3 * H, H), pre + "attention.dense.weight": r(H, H),
               pre + "mlp.dense_h_to_4h.weight": r(F, H), pre + "mlp.dense_h_to_4h.bias": r(F),
               pre + "mlp.dense_4h_to_h.weight": r(H, F), pre + "mlp.dense_4h_to_h.bias": r(H)})
    layers, head = cf.convert_state_dict(sd, cfg, device="cpu")
    w = layers[0]
    assert head["embed_out"] is head["embed_in"]                       # tied: no embed_out.weight in the dict
    assert w["qkv_bias"].shape == (3 * H,) and not w["qkv_bias"].any()  # attention biases absent -> zeros
    assert not w["o_bias"].any() and w["mlp_up_bias"].any()
    assert all(t.dtype == torch.float16 and t.is_contiguous() for t in w.values())
    assert torch.equal(w["qkv_weight"], sd[pre + "attention.query_key_value.weight"].half())
    bad = dict(sd)
    bad[pre + "mlp.dense_h_to_4h.weight"] = r(F + 8, H)
    with pytest.raises(RuntimeError, match="shapes"):
        cf.convert_state_dict(bad, cfg, device="cpu")
    del bad[pre + "input_layernorm.weight"]
    with pytest.raises(RuntimeError):
        cf.convert_state_dict(bad, cfg, device="cpu")


# ---- mirror of the kernel's static split (decode_kernel.cuh: part_begin / part_of)
def part_begin(i, total, parts):
    return (i * total) // parts


def part_of(t, total, parts):
    return ((t + 1) * parts - 1) // total


@pytest.mark.parametrize("total,parts", [(3584, 148), (2048, 148), (10, 4), (64, 148), (1, 148), (4096, 132), (512, 74)])
def test_partition_is_exact_and_invertible(total, parts):
    seen = 0
    for i in range(parts):
        a, b = part_begin(i, total, parts), part_begin(i + 1, total, parts)
        assert a <= b
        for t in range(a, b):
            assert part_of(t, total, parts) == i
        seen += b - a
    assert seen == total
    sizes = [part_begin(i + 1, total, parts) - part_begin(i, total, parts) for i in range(parts)]
    assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("NH,G", [(32, 148), (32, 132), (16, 148), (8, 148), (4, 148)])
@pytest.mark.parametrize("seq", [1, 63, 64, 65, 1000, 4096, 8192, 20000])
def test_attention_item_split_bounds(NH, G, seq):
    """A CTA's items touch at most MAXL = 4 heads, a head is split into at most
    ceil(G / NH) + 2 partials: the sizes the kernel's scratch is laid out for."""
    nch = -(-seq // 128)   # KV_TILE
    T = NH * nch
    pstr = -(-G // NH) + 2
    for c in range(G):
        a, b = part_begin(c, T, G), part_begin(c + 1, T, G)
        if b > a:
            assert (b - 1) // nch - a // nch < 4
    for h in range(NH):
        ia, ib = part_of(h * nch, T, G), part_of((h + 1) * nch - 1, T, G)
        assert ib - ia + 1 <= pstr
        covered = 0
        for c in range(ia, ib + 1):
            a, b = part_begin(c, T, G), part_begin(c + 1, T, G)
            covered += max(0, min(b, (h + 1) * nch) - max(a, h * nch))
        assert covered == nch
