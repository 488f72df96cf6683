"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache, one
function for each part, on the CPU.  It shares no code with lucciola_b200: it reads config.json
with the json module and model.safetensors with its own few lines, and each function restates a
formula of JunkuiZhang/lucciola, cited by file:line of that project.

lucciola's model code cannot be imported or compiled on a CPU: all of its arithmetic is in
__global__ kernels (src/kernels/*.cu) and src/qwen.cc needs <print> and network-fetched headers.
So on the CPU this file rests on the formulas, and tests/golden/ holds outputs of this file only.
On a GPU, tests/test_reference_kernels_gpu.py compiles lucciola's kernel files unchanged and checks
each function of this file against the kernel it restates, to one rounding of the bfloat16 output.

Arithmetic is float64 unless `dtype` says otherwise; the rotation angle is formed in float32 as
lucciola forms it (pos * freq in float, src/kernels/rope.cu:34-37), because at positions in the
thousands that single rounding is larger than anything else in the comparison.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# ---- reading a model folder ----------------------------------------------------------------
def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Container of src/safetensors.cc:51-87: u64 header length, JSON header, data."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        t = torch.frombuffer(bytearray(raw[base + b:base + en]), dtype=kinds[e["dtype"]])
        out[name] = t.reshape(e["shape"])
    return out


def read_model(folder):
    cfg = json.loads((Path(folder) / "config.json").read_text())
    weights = {}
    for f in sorted(Path(folder).glob("*.safetensors")):
        weights.update(read_safetensors(f))
    return cfg, weights


# ---- one function for each part ----------------------------------------------------------------
def embed(ids, table):
    """x_t = E[id_t], unscaled (src/kernels/embedding.cu:22-38)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rms_norm(x, w, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w over the last dimension (src/kernels/rmsnorm.cu:57-97)."""
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def linear(x, w):
    """y[m, n] = sum_k x[m, k] * w[n, k] (src/kernels/linear.cu:24-55; no bias anywhere)."""
    return x @ w.t()


def rope(x, positions, theta):
    """Half rotation of x [T, heads, d]: freq_i = 1 / theta^(2i/d), angle = pos * freq_i in float32,
    (x_i, x_{i+d/2}) <- (x_i cos - x_{i+d/2} sin, x_i sin + x_{i+d/2} cos) (src/kernels/rope.cu:28-60)."""
    d = x.shape[-1]
    half = d // 2
    i = torch.arange(0, d, 2, dtype=torch.float32)
    freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), i / float(d))
    angle = torch.as_tensor(positions, dtype=torch.float32)[:, None] * freq[None, :]      # float32 product
    cos, sin = torch.cos(angle.double()).to(x.dtype)[:, None, :], torch.sin(angle.double()).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def attention(q, k, v, q_positions, k_positions, scale, window=0):
    """Causal grouped-query attention.  q [Tq, nq, d], k and v [Tk, nkv, d].  kv head = q head // (nq // nkv)
    (src/kernels/attention_paged.cu:68); score = q.k * scale; key j allowed iff pos_j <= pos_i
    (src/kernels/flash_attention.cu:183-225), and pos_j > pos_i - window when a window is given;
    softmax over the allowed keys, then the weighted sum of v (src/kernels/flash_attention.cu:246-298, 311-347)."""
    nq, nkv = q.shape[1], k.shape[1]
    rep = nq // nkv
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    qp = torch.as_tensor(q_positions)[:, None]
    kp = torch.as_tensor(k_positions)[None, :]
    ok = kp <= qp
    if window:
        ok = ok & (kp > qp - window)
    s = s.masked_fill(~ok[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, vv)


def swiglu(gate, up):
    """silu(g) * u with silu(x) = x / (1 + exp(-x)) (src/kernels/swiglu.cu:8, 30-36)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def attention_block(x, w, prefix, cfg, positions, window, kv_override=None):
    """Norm, projections, per-head q/k norm before the rotation, rotation, attention, output projection
    (src/qwen.cc:582-742).  Returns the block's output and its (k, v) for layers that share them."""
    nq, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    T = x.shape[0]
    q = linear(x, w[f"{prefix}.q_proj.weight"]).reshape(T, nq, d)
    q = rope(rms_norm(q, w[f"{prefix}.q_norm.weight"], eps), positions, theta)
    if kv_override is None:
        k = linear(x, w[f"{prefix}.k_proj.weight"]).reshape(T, nkv, d)
        v = linear(x, w[f"{prefix}.v_proj.weight"]).reshape(T, nkv, d)
        k = rope(rms_norm(k, w[f"{prefix}.k_norm.weight"], eps), positions, theta)
    else:
        k, v = kv_override
    o = attention(q, k, v, positions, positions, 1.0 / math.sqrt(d), window)
    return linear(o.reshape(T, nq * d), w[f"{prefix}.o_proj.weight"]), (k, v)


def feed_forward(x, w, prefix):
    """down(silu(gate(x)) * up(x)) (src/qwen.cc:762-794)."""
    return linear(swiglu(linear(x, w[f"{prefix}.gate_proj.weight"]), linear(x, w[f"{prefix}.up_proj.weight"])),
                  w[f"{prefix}.down_proj.weight"])


def layer_windows(cfg) -> list[int]:
    """Window of each layer (0: all keys).  lucciola has none; this follows config.json's keys."""
    n = cfg["num_hidden_layers"]
    if cfg.get("layer_types") is not None:
        return [cfg["sliding_window"] if t == "sliding_attention" else 0 for t in cfg["layer_types"]]
    if cfg.get("use_sliding_window"):
        return [cfg["sliding_window"] if i >= cfg["max_window_layers"] else 0 for i in range(n)]
    return [0] * n


def forward(cfg, weights, ids, dtype=torch.float64, calls=None):
    """Logits [T, vocab] of a whole sequence (src/qwen.cc:830-882 without the cache).

    `calls` is the order of the layers: (layer, cache, writes) triples; a call with writes=False uses
    the keys and values that the call which wrote `cache` produced.  Default: each layer once."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["rms_norm_eps"]
    T = len(ids)
    positions = list(range(T))
    windows = layer_windows(cfg)
    x = embed(ids, w["model.embed_tokens.weight"])
    calls = calls or [(i, i, True) for i in range(cfg["num_hidden_layers"])]
    kv_of = {}
    for layer, cache, writes in calls:
        p = f"model.layers.{layer}"
        h = rms_norm(x, w[f"{p}.input_layernorm.weight"], eps)                                  # src/qwen.cc:582-589
        a, kv = attention_block(h, w, f"{p}.self_attn", cfg, positions, windows[layer],
                                None if writes else kv_of[cache])
        if writes:
            kv_of[cache] = kv
        x = x + a                                                                               # src/qwen.cc:742
        h = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps)                         # src/qwen.cc:752-759
        x = x + feed_forward(h, w, f"{p}.mlp")                                                  # src/qwen.cc:797-798
    x = rms_norm(x, w["model.norm.weight"], eps)                                                # src/qwen.cc:851-858
    head = w["lm_head.weight"] if "lm_head.weight" in w and not cfg.get("tie_word_embeddings") else w["model.embed_tokens.weight"]
    return linear(x, head)                                                                      # src/qwen.cc:875-882


# ---- sampling ------------------------------------------------------------------------------
def greedy(logits_row) -> int:
    """Index of the largest logit, the lowest index among equals (src/kernels/argmax.cu:8-59 leaves ties open)."""
    return int(np.argmax(np.asarray(logits_row)))          # numpy returns the first maximal index


_M64 = (1 << 64) - 1


def _mix64(x: int) -> int:
    x ^= x >> 30; x = (x * 0xBF58476D1CE4E5B9) & _M64
    x ^= x >> 27; x = (x * 0x94D049BB133111EB) & _M64
    x ^= x >> 31
    return x


def bits_to_uniform(bits23):
    """(b + 0.5) / 2^23 in float32 for 23-bit b (a number or an array): exact, and strictly inside (0, 1)."""
    return (np.asarray(bits23, dtype=np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)


def hash_uniform(key: int, counter: int, i: int) -> np.float32:
    """The uniform number in (0, 1) that the temperature sampler uses for vocabulary index i."""
    x = _mix64((key + 0x9E3779B97F4A7C15 * (counter + 1)) & _M64)
    x = _mix64(x ^ ((0xD6E8FEB86659FD93 * (i + 1)) & _M64))
    return np.float32(bits_to_uniform(x >> 41))


def request_key(seed: int, request_index: int) -> int:
    return _mix64((seed & _M64) ^ _mix64((request_index + 0x632BE59BD9B4E019) & _M64))


def temperature_sample(logits_row, temperature: float, key: int, counter: int) -> int:
    """Gumbel-max draw from softmax(logits / T): argmax_i(logits_i / T - log(-log(u_i))), float32 as on the GPU."""
    if not temperature > 0:
        return greedy(logits_row)
    l = np.asarray(logits_row, dtype=np.float32)
    u = np.array([hash_uniform(key, counter, i) for i in range(l.shape[0])], dtype=np.float32)
    s = l * np.float32(1.0 / np.float32(temperature)) - np.log(-np.log(u))
    return int(np.argmax(s))


def generate(cfg, weights, prompt, max_new_tokens, temperature=0.0, key=0, eos=(), dtype=torch.float64):
    """Token by token from whole-sequence recomputation: the slowest possible generation loop."""
    ids = list(prompt)
    out = []
    for n in range(max_new_tokens):
        row = forward(cfg, weights, ids, dtype)[-1]
        t = temperature_sample(row.float().numpy(), temperature, key, n) if temperature > 0 else greedy(row)
        out.append(t)
        ids.append(t)
        if t in eos:
            break
    return out
