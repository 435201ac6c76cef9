"""Tensor-parallel decode on the GPUs of one box (one process per GPU).

The reference is single-GPU (it pins cuda:0, include/5090/pythia_6b9/pythia_kernel_dispatch.cu:31)
and has no communication backend; this mode is new.  Partition, per layer:

  * attention heads: rows [h*3D, (h+1)*3D) of the interleaved QKV weight and bias, the
    head's columns of the KV cache, and the matching COLUMNS of the dense weight;
  * MLP: rows of the up-projection (+ bias) and the matching COLUMNS of the down-projection;
  * LayerNorm parameters, dense bias, down bias and the hidden state are replicated.

Each rank computes LayerNorm redundantly and produces a partial attention + MLP
output of full width; ONE all-reduce (sum) of that [hidden] vector per layer combines
them, after which every rank adds the residual and the two replicated biases exactly
once.  The LM head is sharded by vocabulary rows; the ranks exchange their (max logit,
index) pairs and pick the same winner.

Two data paths: `fused=True` (default) runs the whole token as one launch per rank and
does the all-reduce inside the kernel -- every CTA stores its fp32 partial rows into the
peers' exchange buffers over NVLink, publishes a flag and sums the N partials in rank
order (deterministic, identical on all ranks); `fused=False` is the baseline with one
NCCL all-reduce of the fp16 partial per layer between two launches.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ._lib import CfDecoderConfig, CfDims, CfHeadWeights, check, lib
from .api import _req, _wrap
from .decoder import _F32View, _IntView, layer_weights_struct, rope_table


def shard_dims(full: CfDims, size: int) -> CfDims:
    if full.heads % size or full.ffn % size or full.vocab % (8 * size):
        raise RuntimeError(f"heads {full.heads}, ffn {full.ffn} and vocab {full.vocab} must divide by tp size {size}")
    d = CfDims()
    d.hidden, d.head_dim, d.rotary = full.hidden, full.head_dim, full.rotary
    d.heads, d.ffn, d.vocab = full.heads // size, full.ffn // size, full.vocab // size
    return d


def shard_layer_weights(w: Dict[str, torch.Tensor], full: CfDims, rank: int, size: int) -> Dict[str, torch.Tensor]:
    """Rank `rank`'s contiguous copies of one layer's tensors."""
    D = full.head_dim
    nh, f = full.heads // size, full.ffn // size
    q0, q1 = rank * nh * 3 * D, (rank + 1) * nh * 3 * D
    c0, c1 = rank * nh * D, (rank + 1) * nh * D
    f0, f1 = rank * f, (rank + 1) * f
    return {
        "qkv_weight": w["qkv_weight"][q0:q1].contiguous(),
        "qkv_bias": w["qkv_bias"][q0:q1].contiguous(),
        "o_weight": w["o_weight"][:, c0:c1].contiguous(),
        "o_bias": w["o_bias"].reshape(-1),
        "ln_weight": w["ln_weight"].reshape(-1), "ln_bias": w["ln_bias"].reshape(-1),
        "post_ln_weight": w["post_ln_weight"].reshape(-1), "post_ln_bias": w["post_ln_bias"].reshape(-1),
        "mlp_up_weight": w["mlp_up_weight"][f0:f1].contiguous(),
        "mlp_up_bias": w["mlp_up_bias"][f0:f1].contiguous(),
        "mlp_down_weight": w["mlp_down_weight"][:, f0:f1].contiguous(),
        "mlp_down_bias": w["mlp_down_bias"].reshape(-1),
    }


def shard_head_weights(head: Dict[str, torch.Tensor], full: CfDims, rank: int, size: int) -> Dict[str, torch.Tensor]:
    v = full.vocab // size
    out = dict(head)
    out["embed_out"] = head["embed_out"][rank * v:(rank + 1) * v].contiguous()
    return out


def shard_cache(cache: torch.Tensor, full: CfDims, rank: int, size: int) -> torch.Tensor:
    """[rows, heads*D] -> this rank's [rows, heads/size*D] columns."""
    w = (full.heads // size) * full.head_dim
    return cache[:, rank * w:(rank + 1) * w].contiguous()


class TPDecoder:
    """Greedy decoder over already-sharded tensors; all ranks call the same methods.

    local_layers / local_head / local_caches are this rank's shards (see the shard_*
    helpers).  `group` is a torch.distributed process group with the NCCL backend.
    """

    def __init__(self, full_dims: CfDims, local_layers: Sequence[Dict[str, torch.Tensor]],
                 local_head: Dict[str, torch.Tensor], local_caches: Sequence, max_seq: int,
                 group: Optional[dist.ProcessGroup] = None, use_graph: bool = True, fused: bool = True):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.full = full_dims
        self.dims = shard_dims(full_dims, self.size)
        self.layers, self.head, self.caches = list(local_layers), local_head, list(local_caches)
        self.max_seq = int(max_seq)
        self.device = local_head["embed_in"].device
        self.cos, self.sin = rope_table(self.max_seq, full_dims.rotary, self.device)
        cfg = CfDecoderConfig()
        cfg.dims = self.dims
        cfg.n_layers = len(self.layers)
        cfg.max_seq_len = self.max_seq
        cfg.tp_size, cfg.tp_rank = self.size, self.rank
        cfg.cos_table, cfg.sin_table = self.cos.data_ptr(), self.sin.data_ptr()
        h = C.c_int64(0)
        check(lib.cf_decoder_create(C.byref(cfg), C.byref(h)))
        self.handle = h.value
        kvw = self.dims.heads * self.dims.head_dim
        for i, (w, (k, v)) in enumerate(zip(self.layers, self.caches)):
            if tuple(k.shape) != (self.max_seq, kvw) or tuple(v.shape) != (self.max_seq, kvw):
                raise RuntimeError(f"layer {i}: local caches must be [{self.max_seq}, {kvw}]")
            check(lib.cf_decoder_set_layer(self.handle, i, C.byref(layer_weights_struct(self.dims, w)),
                                           _req(k, "k_cache", k.numel()), _req(v, "v_cache", v.numel())))
        hw = CfHeadWeights()
        hw.embed_in = _req(local_head["embed_in"], "embed_in", local_head["embed_in"].numel())
        hw.final_ln_weight = _req(local_head["final_ln_weight"], "final_ln_weight", self.dims.hidden)
        hw.final_ln_bias = _req(local_head["final_ln_bias"], "final_ln_bias", self.dims.hidden)
        hw.embed_out = _req(local_head["embed_out"], "embed_out", self.dims.vocab * self.dims.hidden)
        hw.vocab_offset = self.rank * self.dims.vocab
        check(lib.cf_decoder_set_head(self.handle, C.byref(hw)))
        check(lib.cf_decoder_finalize(self.handle))
        p = [C.c_void_p() for _ in range(7)]
        check(lib.cf_decoder_state(self.handle, *[C.byref(x) for x in p]))
        dev = self.device
        self.token = torch.as_tensor(_IntView(p[0].value, (1,)), device=dev)
        self.seq_len = torch.as_tensor(_IntView(p[1].value, (1,)), device=dev)
        self.logits = torch.as_tensor(_F32View(p[2].value, (self.dims.vocab,)), device=dev)  # this rank's rows
        self.hidden = _wrap(p[3].value, (1, self.dims.hidden), dev)
        self.partial = _wrap(p[4].value, (self.dims.hidden,), dev)
        self.shard_max = torch.as_tensor(_F32View(p[5].value, (1,)), device=dev)
        self.shard_idx = torch.as_tensor(_IntView(p[6].value, (1,)), device=dev)
        self.all_max = torch.empty(self.size, dtype=torch.float32, device=dev)
        self.all_idx = torch.empty(self.size, dtype=torch.int32, device=dev)
        self.use_graph = use_graph
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self.fused = fused
        if fused:
            # exchange buffers of all ranks mapped into each other (CUDA IPC over NVLink peer access)
            mine = (C.c_char * 64)()
            check(lib.cf_decoder_tp_export(self.handle, C.cast(mine, C.c_void_p)))
            t = torch.frombuffer(bytearray(mine.raw), dtype=torch.uint8).to(dev)
            allh = torch.empty(64 * self.size, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(allh, t, group=self.group)
            raw = bytes(allh.cpu().numpy().tobytes())
            check(lib.cf_decoder_tp_connect(self.handle, C.cast(C.create_string_buffer(raw, len(raw)), C.c_void_p)))
            dist.barrier(group=self.group)
        self.launches_per_token = 1 if fused else 2 * len(self.layers) + 3  # ours (NCCL's kernels not counted)

    def reset(self, seq_len: int, token: int) -> None:
        self.seq_len.fill_(int(seq_len))
        self.token.fill_(int(token))

    def _enqueue(self) -> None:
        st = torch.cuda.current_stream().cuda_stream
        if self.fused:
            check(lib.cf_decoder_step(self.handle, st))
            return
        for l in range(len(self.layers)):
            check(lib.cf_decoder_layer_partial(self.handle, l, st))
            dist.all_reduce(self.partial, group=self.group)
            check(lib.cf_decoder_layer_finish(self.handle, l, st))
        check(lib.cf_decoder_tail(self.handle, st))
        dist.all_gather_into_tensor(self.all_max, self.shard_max, group=self.group)
        dist.all_gather_into_tensor(self.all_idx, self.shard_idx, group=self.group)
        check(lib.cf_decoder_select_token(self.handle, self.all_max.data_ptr(), self.all_idx.data_ptr(), st))

    def capture(self) -> None:
        seq0, tok0 = self.seq_len.clone(), self.token.clone()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._enqueue()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._enqueue()
        self._graph = g
        self.seq_len.copy_(seq0)
        self.token.copy_(tok0)

    def step(self) -> None:
        if self.use_graph:
            if self._graph is None:
                self.capture()
            self._graph.replay()
        else:
            self._enqueue()

    def status(self) -> int:
        """This decoder's device status word (0 = every launch so far ended normally; 7 = a peer never
        answered within the kernel's bounded wait).  A blocking 4-byte read; not cleared."""
        st = C.c_int(0)
        check(lib.cf_decoder_status(self.handle, C.byref(st)))
        return st.value

    def generate(self, first_token: int, seq_len: int, n_tokens: int) -> List[int]:
        """Greedy rollout with one host read per token.  The status word is checked after every token:
        a rank whose peer stopped answering would otherwise decode on with wrong tokens.  Callers that
        drive step() themselves should poll status() the same way."""
        self.reset(seq_len, first_token)
        out = []
        for _ in range(n_tokens):
            self.step()
            out.append(int(self.token.item()))
            code = self.status()
            if code != 0:
                raise RuntimeError(f"clusterfusion_b200: tensor-parallel decode stopped with device status {code} "
                                   f"on rank {self.rank} after {len(out)} tokens (7 = a peer never answered)")
        return out

    def close(self) -> None:
        if self.handle:
            self._graph = None
            check(lib.cf_decoder_destroy(self.handle))
            self.handle = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
