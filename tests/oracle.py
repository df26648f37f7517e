"""Independent NumPy restatement of the decoder graph semantics (the exact-match oracle).

It shares no code with the runtime: weights are read straight from the ONNX initializers by name,
attention is dense over the whole prefix and recomputed from scratch for every new token (no KV
cache, no paging, no packing), greedy search is a plain argmax.  It plays the role the reference
binary would play if it could run here.
"""
import json
import os

import numpy as np

from onnxruntime_genai_b200.utils import onnx_proto as op


def _f32(lm, name):
    t = lm.info(name)
    a = lm.array(name)
    if t.dtype == op.BFLOAT16:
        return (a.astype(np.uint32) << 16).view(np.float32)
    return a.astype(np.float32)


class NumpyLlama:
    def __init__(self, model_dir):
        with open(os.path.join(model_dir, "genai_config.json")) as f:
            cfg = json.load(f)
        d = cfg["model"]["decoder"]
        self.L, self.H = d["num_hidden_layers"], d["hidden_size"]
        self.nh, self.nkv, self.hd = d["num_attention_heads"], d["num_key_value_heads"], d["head_size"]
        self.eos = cfg["model"]["eos_token_id"]
        lm = op.LoadedModel(os.path.join(model_dir, d["filename"]))
        self.eps = [n for n in lm.model.nodes if "input_layernorm" in n.name][0].attrs["epsilon"]
        g = lambda n: _f32(lm, n)
        self.embed = g("model.embed_tokens.weight")
        self.cos, self.sin = g("cos_cache"), g("sin_cache")
        self.layers = []
        for i in range(self.L):
            p = f"model.layers.{i}."
            self.layers.append(dict(ln1=g(p + "input_layernorm.weight"), qkv=g(p + "attn.qkv_proj.MatMul.weight"),
                                    o=g(p + "attn.o_proj.MatMul.weight"), ln2=g(p + "post_attention_layernorm.weight"),
                                    gu=g(p + "mlp.gate_up_proj.MatMul.weight"), down=g(p + "mlp.down_proj.MatMul.weight")))
        self.fnorm = g(f"model.layers.{self.L}.final_norm_layernorm.weight")
        self.head = g("lm_head.MatMul.weight")

    def _rms(self, x, w):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + self.eps) * w

    def _rope(self, x, pos):  # x [S, heads, hd]
        half = self.hd // 2
        c, s = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        x1, x2 = x[..., :half], x[..., half:]
        return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    def logits(self, ids):
        """ids: 1-D token list; returns the logits of the last position."""
        S = len(ids)
        pos = np.arange(S)
        h = self.embed[np.asarray(ids)]
        G = self.nh // self.nkv
        for lw in self.layers:
            x = self._rms(h, lw["ln1"])
            qkv = x @ lw["qkv"]
            q = qkv[:, :self.nh * self.hd].reshape(S, self.nh, self.hd)
            k = qkv[:, self.nh * self.hd:(self.nh + self.nkv) * self.hd].reshape(S, self.nkv, self.hd)
            v = qkv[:, (self.nh + self.nkv) * self.hd:].reshape(S, self.nkv, self.hd)
            q, k = self._rope(q, pos), self._rope(k, pos)
            k, v = np.repeat(k, G, axis=1), np.repeat(v, G, axis=1)
            s = np.einsum("qhd,khd->hqk", q, k) / np.sqrt(self.hd)
            s = np.where(np.tril(np.ones((S, S), bool))[None], s, -np.inf)
            s = s - s.max(-1, keepdims=True)
            p = np.exp(s)
            p /= p.sum(-1, keepdims=True)
            a = np.einsum("hqk,khd->qhd", p, v).reshape(S, self.nh * self.hd)
            h = h + a @ lw["o"]
            x = self._rms(h, lw["ln2"])
            gu = x @ lw["gu"]
            inter = gu.shape[-1] // 2
            g_, u_ = gu[:, :inter], gu[:, inter:]
            h = h + ((g_ / (1 + np.exp(-g_))) * u_) @ lw["down"]
        return self._rms(h[-1], self.fnorm) @ self.head

    def greedy(self, prompt, new_tokens):
        ids = list(prompt)
        for _ in range(new_tokens):
            ids.append(int(np.argmax(self.logits(ids))))
        return ids
