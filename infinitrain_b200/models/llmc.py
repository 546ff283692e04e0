"""llm.c ``.bin`` weight files for GPT-2 and LLaMA-3: read (sharded per TP / PP rank) and write.

Reference: example/gpt2/checkpoint_loader.cc:39-428, example/llama3/checkpoint_loader.cc:37-347,
example/common/utils.cc:27-62.

GPT-2 file: 256 x int32 header (magic 20240326, version 3 = fp32, block_size, vocab_size, n_layer,
n_head, n_embd, padded_vocab_size), then fp32 tensors grouped by KIND across layers:
wte [Vp, C], wpe [block, C], ln_1.w [L, C], ln_1.b, c_attn.w [L, 3C, C] (rows Q|K|V), c_attn.b,
attn.c_proj.w [L, C, C], attn.c_proj.b, ln_2.w, ln_2.b, c_fc.w [L, 4C, C], c_fc.b,
mlp.c_proj.w [L, C, 4C], mlp.c_proj.b, ln_f.w, ln_f.b.  No lm_head (tied to wte).

LLaMA-3 file: 256 x 4-byte header (magic 20240803, version 3, block_size, vocab_size, n_layer, n_head,
n_kv_head, n_embd, ffn_dim_multiplier (float), multiple_of, norm_eps (float), rope_theta (float),
use_scaled_rope, max_gen_bs, version_major, version_minor), then fp32: wte [V, C], ln_1.w [L, C],
c_attn.w [L, (H + 2 KV) D, C] (rows Q|K|V), attn.c_proj.w [L, C, C], ln_2.w, c_fc.w [L, F, C],
c_fc2.w [L, F, C], mlp.c_proj.w [L, C, F], ln_f.w [C], lm_head.w [V, C].

Sharding at load: column-parallel weights take a ROW block, row-parallel weights a COLUMN block, the
fused QKV takes ``[q_r | k_r | v_r]``; a pipeline rank reads only its layers (state-dict layer indices
are stage-local).
"""
from __future__ import annotations

import struct
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..nn.transformer import TransformerConfig, TransformerModel
from ..parallel import global_env as genv

kGpt2Magic, kGpt2Fp32Version = 20240326, 3
kLlama3Magic, kLlama3Fp32Version = 20240803, 3


def _round_up(x, m):
    return (x + m - 1) // m * m


# --------------------------------------------------------------------------- full-model tensors <-> file
def _gpt2_layout(cfg: TransformerConfig, Vp: int):
    L, C = cfg.n_layer, cfg.n_embd
    F = cfg.ffn_hidden()
    return [("wte", (Vp, C)), ("wpe", (cfg.block_size, C)), ("ln_1.weight", (L, C)), ("ln_1.bias", (L, C)),
            ("attn.c_attn.weight", (L, 3 * C, C)), ("attn.c_attn.bias", (L, 3 * C)),
            ("attn.c_proj.weight", (L, C, C)), ("attn.c_proj.bias", (L, C)), ("ln_2.weight", (L, C)),
            ("ln_2.bias", (L, C)), ("mlp.c_fc.weight", (L, F, C)), ("mlp.c_fc.bias", (L, F)),
            ("mlp.c_proj.weight", (L, C, F)), ("mlp.c_proj.bias", (L, C)), ("ln_f.weight", (C,)), ("ln_f.bias", (C,))]


def _llama3_layout(cfg: TransformerConfig):
    L, C, V = cfg.n_layer, cfg.n_embd, cfg.vocab_size
    D = cfg.head_dim()
    F = cfg.ffn_hidden()
    Q = (cfg.n_head + 2 * cfg.n_kv_head) * D
    return [("wte", (V, C)), ("ln_1.weight", (L, C)), ("attn.c_attn.weight", (L, Q, C)),
            ("attn.c_proj.weight", (L, C, C)), ("ln_2.weight", (L, C)), ("mlp.c_fc.weight", (L, F, C)),
            ("mlp.c_fc2.weight", (L, F, C)), ("mlp.c_proj.weight", (L, C, F)), ("ln_f.weight", (C,)),
            ("lm_head", (V, C))]


def _full_to_kinds(cfg, full: Dict[str, torch.Tensor], layout) -> Dict[str, np.ndarray]:
    """Global state dict (keys ``transformer.h.<i>.attn...``) -> per-kind stacked arrays."""
    out = {}
    for kind, shape in layout:
        if kind == "wte":
            w = full["transformer.wte.weight"].float().numpy()
            arr = np.zeros(shape, dtype=np.float32)
            arr[: w.shape[0]] = w
        elif kind == "wpe":
            arr = full["transformer.wpe.weight"].float().numpy()
        elif kind in ("ln_f.weight", "ln_f.bias"):
            arr = full[f"transformer.{kind}"].float().numpy()
        elif kind == "lm_head":
            arr = full["lm_head.weight"].float().numpy()
        else:
            arr = np.stack([full[f"transformer.h.{i}.{kind}"].float().numpy() for i in range(cfg.n_layer)])
        out[kind] = np.ascontiguousarray(arr, dtype=np.float32).reshape(shape)
    return out


def write_gpt2_llmc(path: str, cfg: TransformerConfig, full_state: Dict[str, torch.Tensor],
                    padded_vocab_size: Optional[int] = None) -> None:
    Vp = padded_vocab_size or _round_up(cfg.original_vocab_size, 128)
    header = np.zeros(256, dtype=np.int32)
    header[:8] = [kGpt2Magic, kGpt2Fp32Version, cfg.block_size, cfg.original_vocab_size, cfg.n_layer, cfg.n_head,
                  cfg.n_embd, Vp]
    layout = _gpt2_layout(cfg, Vp)
    kinds = _full_to_kinds(cfg, full_state, layout)
    with open(path, "wb") as f:
        f.write(header.tobytes())
        for kind, _ in layout:
            f.write(kinds[kind].tobytes())


def write_llama3_llmc(path: str, cfg: TransformerConfig, full_state: Dict[str, torch.Tensor]) -> None:
    header = bytearray(1024)
    struct.pack_into("<8i", header, 0, kLlama3Magic, kLlama3Fp32Version, cfg.block_size, cfg.vocab_size, cfg.n_layer,
                     cfg.n_head, cfg.n_kv_head, cfg.n_embd)
    struct.pack_into("<f", header, 32, float(cfg.ffn_dim_multiplier or 0.0))
    struct.pack_into("<i", header, 36, cfg.multiple_of)
    struct.pack_into("<f", header, 40, float(cfg.norm_eps))
    struct.pack_into("<f", header, 44, float(cfg.rope_theta))
    struct.pack_into("<4i", header, 48, int(cfg.use_scaled_rope), cfg.max_gen_batch_size, 3, 1)
    layout = _llama3_layout(cfg)
    kinds = _full_to_kinds(cfg, full_state, layout)
    with open(path, "wb") as f:
        f.write(bytes(header))
        for kind, _ in layout:
            f.write(kinds[kind].tobytes())


# --------------------------------------------------------------------------- reading
def read_gpt2_header(path: str) -> Tuple[TransformerConfig, int]:
    h = np.fromfile(path, dtype=np.int32, count=256)
    if h[0] != kGpt2Magic:
        raise ValueError(f"bad GPT-2 llm.c magic {h[0]}")
    if h[1] != kGpt2Fp32Version:
        raise ValueError(f"unsupported GPT-2 llm.c version {h[1]} (only 3 = fp32)")
    tp = genv.GetTensorParallelSize()
    vocab, Vp = int(h[3]), int(h[7])
    cfg = TransformerConfig.GPT2(block_size=int(h[2]), original_vocab_size=vocab, vocab_size=Vp if tp > 1 else vocab,
                                 n_layer=int(h[4]), n_head=int(h[5]), n_kv_head=int(h[5]), n_embd=int(h[6]))
    return cfg, Vp


def read_llama3_header(path: str) -> TransformerConfig:
    raw = open(path, "rb").read(1024)
    magic, version, block, vocab, L, H, KV, C = struct.unpack_from("<8i", raw, 0)
    if magic != kLlama3Magic:
        raise ValueError(f"bad LLaMA-3 llm.c magic {magic}")
    if version != kLlama3Fp32Version:
        raise ValueError(f"unsupported LLaMA-3 llm.c version {version}")
    (mult,) = struct.unpack_from("<f", raw, 32)
    (multiple_of,) = struct.unpack_from("<i", raw, 36)
    eps, theta = struct.unpack_from("<2f", raw, 40)
    scaled, max_gen = struct.unpack_from("<2i", raw, 48)
    return TransformerConfig.LLaMA3(block_size=block, vocab_size=vocab, original_vocab_size=vocab, n_layer=L, n_head=H,
                                    n_kv_head=KV, n_embd=C, ffn_dim_multiplier=mult if mult > 0 else None,
                                    multiple_of=multiple_of, norm_eps=eps, rope_theta=theta,
                                    use_scaled_rope=bool(scaled), max_gen_batch_size=max_gen)


def _kind_views(path: str, layout):
    mm = np.memmap(path, dtype=np.float32, mode="r", offset=1024)
    out, off = {}, 0
    for kind, shape in layout:
        n = int(np.prod(shape))
        out[kind] = mm[off:off + n].reshape(shape)
        off += n
    if off > mm.size:
        raise ValueError("llm.c weight file is truncated")
    return out


def _rows(a, r, n):   # column-parallel: block of rows
    k = a.shape[0] // n
    return a[r * k:(r + 1) * k]


def _cols(a, r, n):   # row-parallel: block of columns
    k = a.shape[1] // n
    return a[:, r * k:(r + 1) * k]


def _qkv_rows(a, r, n, q_rows, kv_rows):
    """[q_r | k_r | v_r] of a fused projection whose rows are Q (q_rows) | K (kv_rows) | V (kv_rows)."""
    q, k, v = a[:q_rows], a[q_rows:q_rows + kv_rows], a[q_rows + kv_rows:]
    return np.concatenate([_rows(q, r, n), _rows(k, r, n), _rows(v, r, n)], axis=0)


def _fill(model: TransformerModel, kinds, cfg: TransformerConfig, has_bias: bool):
    tp, tr = genv.GetTensorParallelSize(), genv.GetTensorParallelRank()
    D = cfg.head_dim()
    q_rows, kv_rows = cfg.n_head * D, cfg.n_kv_head * D
    layers = [l for (s, e) in sorted(model.stage_info.layer_ranges_per_chunk) for l in range(s, e)]
    sd = model.StateDict()

    def put(key, arr):
        t = sd[key]
        with torch.no_grad():
            t.copy_(torch.from_numpy(np.array(arr, dtype=np.float32)).to(t.dtype))

    if model.stage_info.is_first_stage:
        wte = kinds["wte"]
        V = cfg.vocab_size
        full = wte[:V] if wte.shape[0] >= V else np.concatenate([wte, np.zeros((V - wte.shape[0], wte.shape[1]), np.float32)])
        put("transformer.wte.weight", _rows(full, tr, tp))
        if "wpe" in kinds:
            put("transformer.wpe.weight", kinds["wpe"])
    for local, g in enumerate(layers):
        p = f"transformer.h.{local}."
        put(p + "ln_1.weight", kinds["ln_1.weight"][g])
        put(p + "ln_2.weight", kinds["ln_2.weight"][g])
        put(p + "attn.c_attn.weight", _qkv_rows(kinds["attn.c_attn.weight"][g], tr, tp, q_rows, kv_rows))
        put(p + "attn.c_proj.weight", _cols(kinds["attn.c_proj.weight"][g], tr, tp))
        put(p + "mlp.c_fc.weight", _rows(kinds["mlp.c_fc.weight"][g], tr, tp))
        put(p + "mlp.c_proj.weight", _cols(kinds["mlp.c_proj.weight"][g], tr, tp))
        if "mlp.c_fc2.weight" in kinds:
            put(p + "mlp.c_fc2.weight", _rows(kinds["mlp.c_fc2.weight"][g], tr, tp))
        if has_bias:
            put(p + "ln_1.bias", kinds["ln_1.bias"][g])
            put(p + "ln_2.bias", kinds["ln_2.bias"][g])
            put(p + "attn.c_attn.bias", _qkv_rows(kinds["attn.c_attn.bias"][g][:, None], tr, tp, q_rows, kv_rows)[:, 0])
            put(p + "attn.c_proj.bias", kinds["attn.c_proj.bias"][g])
            put(p + "mlp.c_fc.bias", _rows(kinds["mlp.c_fc.bias"][g][:, None], tr, tp)[:, 0])
            put(p + "mlp.c_proj.bias", kinds["mlp.c_proj.bias"][g])
    if model.stage_info.is_last_stage:
        put("transformer.ln_f.weight", kinds["ln_f.weight"])
        if has_bias:
            put("transformer.ln_f.bias", kinds["ln_f.bias"])
        if "lm_head" in kinds:
            put("lm_head.weight", _rows(kinds["lm_head"], tr, tp))
        elif not (cfg.tie_weights and genv.GetPipelineParallelSize() == 1):
            wte = kinds["wte"]
            V = cfg.vocab_size
            full = wte[:V] if wte.shape[0] >= V else np.concatenate([wte, np.zeros((V - wte.shape[0], wte.shape[1]), np.float32)])
            put("lm_head.weight", _rows(full, tr, tp))


def GPT2FromLLMC(path: str, **config_overrides) -> TransformerModel:
    cfg, Vp = read_gpt2_header(path)
    for k, v in config_overrides.items():
        setattr(cfg, k, v)
    model = TransformerModel(cfg)
    _fill(model, _kind_views(path, _gpt2_layout(cfg, Vp)), cfg, has_bias=True)
    return model


def LLaMA3FromLLMC(path: str, **config_overrides) -> TransformerModel:
    cfg = read_llama3_header(path)
    for k, v in config_overrides.items():
        setattr(cfg, k, v)
    model = TransformerModel(cfg)
    _fill(model, _kind_views(path, _llama3_layout(cfg)), cfg, has_bias=False)
    return model


def full_state_dict(model: TransformerModel) -> Dict[str, torch.Tensor]:
    """State dict of an unpartitioned model with detached CPU tensors (input of the writers)."""
    return {k: v.detach().cpu() for k, v in model.StateDict().items()}
