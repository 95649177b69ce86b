"""CPU restatement of one Qwen3 W8A8 forward pass, assembled from the oracle's operators in the order of the
reference's forward (crates/inferrous-qwen3/src/gpu.rs:528-817; tools/reference.py:75-121).  Test code only."""
from __future__ import annotations

import numpy as np

from oracle import oracle
from tests.util import to_host


def export(weights) -> dict:
    """Device weights of inferrous_b200.qwen3.Qwen3Weights -> numpy."""
    def m(matrix):
        return matrix.w.cpu().numpy(), matrix.scale.cpu().numpy()

    return dict(
        config=weights.config,
        embedding=oracle.bf16_bits(to_host(weights.embedding)),
        rope=weights.rope.cpu().numpy(),
        final_gain=to_host(weights.final_gain),
        head=m(weights.head) if weights.head is not None else None,
        head_bf16=oracle.bf16_bits(to_host(weights.head_bf16)) if weights.head_bf16 is not None else None,
        layers=[dict(norm1=to_host(l.norm1), norm2=to_host(l.norm2), qnorm=l.qnorm.cpu().numpy(), knorm=l.knorm.cpu().numpy(),
                     qkv=m(l.qkv), o=m(l.o), gate_up=m(l.gate_up), down=m(l.down)) for l in weights.layers],
    )


class OracleModel:
    def __init__(self, exported: dict):
        self.p = exported
        c = exported["config"]
        self.c = c
        self.k = [np.zeros((c.context, c.kv_heads, 128), np.uint16) for _ in range(c.layers)]
        self.v = [np.zeros((c.context, c.kv_heads, 128), np.uint16) for _ in range(c.layers)]

    def project(self, x, matrix, residual=None):
        q, s = oracle.quantize(x)
        return oracle.linear(q, s, matrix[0], matrix[1], residual_in=residual)

    def forward(self, ids, position: int):
        """Returns (final hidden rows, logits of the last row)."""
        c, p = self.c, self.p
        rows = len(ids)
        hidden = oracle.embedding(ids, p["embedding"])
        for index, layer in enumerate(p["layers"]):
            qkv = self.project(oracle.rmsnorm(hidden, layer["norm1"], c.eps), layer["qkv"])
            nq, nk = c.q_heads * 128, c.kv_heads * 128
            q = oracle.head_norm_rope(qkv[:, :nq].reshape(rows, c.q_heads, 128), layer["qnorm"], p["rope"], position, c.eps)
            k = oracle.head_norm_rope(qkv[:, nq:nq + nk].reshape(rows, c.kv_heads, 128), layer["knorm"], p["rope"], position, c.eps)
            self.k[index][position:position + rows] = oracle.bf16_bits(k)
            self.v[index][position:position + rows] = oracle.bf16_bits(qkv[:, nq + nk:].reshape(rows, c.kv_heads, 128))
            a = oracle.attention(q, self.k[index], self.v[index], position).reshape(rows, nq)
            residual = self.project(a, layer["o"], residual=hidden)[1]
            gu = self.project(oracle.rmsnorm(residual, layer["norm2"], c.eps), layer["gate_up"])
            act = np.stack([oracle.swiglu(gu[r, :c.intermediate], gu[r, c.intermediate:])[0] for r in range(rows)])
            hidden = self.project(act, layer["down"], residual=residual)[1]
        last = oracle.rmsnorm(hidden[-1:], p["final_gain"], c.eps)
        if p.get("head_bf16") is not None:  # the reference's own head: bf16 weights, its summation order
            return hidden, oracle.head(last[0], p["head_bf16"])
        logits = self.project(last, p["head"])
        return hidden, logits[0]

    def generate(self, prompt_ids, max_tokens: int):
        tokens, ids, position = [], list(prompt_ids), 0
        for _ in range(max_tokens):
            _, logits = self.forward(np.array(ids, np.uint32), position)
            token = int(np.flatnonzero(logits == logits.max())[0])
            tokens.append(token)
            position += len(ids)
            ids = [token]
        return tokens
