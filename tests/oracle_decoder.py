"""CPU oracle of the int4 decoder: the same operator sequence as yscv_b200/decoder.py,
composed from the oracle's restatements of the reference primitives (RMSNorm, rotate-half
RoPE, GQA attention with the causal limit, scalar SiLU, packed-int4 matmul with the
runner's GEMV/GEMM threshold, argmax-last). Test infrastructure only."""
import numpy as np


class OracleDecoder:
    def __init__(self, oracle, cfg, n_layers, weights, embedding, lm_head, batch, threads=8, kv_int8=False):
        """weights[l][name] = (packed uint8 [n,k/2], scales f32 [n,k/g]) for
        name in q,k,v,o,gate,up,down (unsharded)."""
        self.o, self.cfg, self.n_layers, self.w = oracle, cfg, n_layers, weights
        self.emb, self.lm_head, self.batch, self.threads = embedding, lm_head, batch, threads
        # KvDtype::I8 (kv_cache.rs:8-90): rows are quantised when appended and dequantised when
        # read, so the cache below holds the dequantised values
        self.kv_int8 = kv_int8
        self.k = [[np.zeros((0, cfg.n_kv * cfg.head_dim), np.float32) for _ in range(batch)] for _ in range(n_layers)]
        self.v = [[np.zeros((0, cfg.n_kv * cfg.head_dim), np.float32) for _ in range(batch)] for _ in range(n_layers)]
        self.pos = 0

    def _lin(self, w, x):
        packed, scales = w
        n, k = packed.shape[0], packed.shape[1] * 2
        return self.o.exec_matmul_int4(np.ascontiguousarray(packed).ravel(), np.ascontiguousarray(scales).ravel(),
                                       x, x.shape[0], n, k, self.cfg.group_size, threads=self.threads)

    def forward(self, tokens, seq):
        """tokens: int [batch, seq]. Returns (logits [batch, vocab], next tokens [batch])."""
        c, o, B = self.cfg, self.o, self.batch
        H, d = c.hidden, c.head_dim
        gamma = np.ones(H, np.float32)
        x = self.emb[tokens.reshape(-1)].astype(np.float32)  # [B*seq, H]
        for l in range(self.n_layers):
            w = self.w[l]
            h = o.rms_norm(x, gamma, c.eps)
            q, k, v = self._lin(w["q"], h), self._lin(w["k"], h), self._lin(w["v"], h)
            attn = np.empty((B * seq, c.n_q * d), np.float32)
            for b in range(B):
                sl = slice(b * seq, (b + 1) * seq)
                qb, kb = o.rope(q[sl].ravel(), k[sl].ravel(), c.n_q, c.n_kv, d, seq, self.pos, c.rope_theta)
                new_k, new_v = kb.reshape(seq, -1), v[sl]
                if self.kv_int8:
                    new_k = o.kv_dequantise_i8(*o.kv_append_i8(new_k))
                    new_v = o.kv_dequantise_i8(*o.kv_append_i8(new_v))
                self.k[l][b] = np.concatenate([self.k[l][b], new_k])
                self.v[l][b] = np.concatenate([self.v[l][b], new_v])
                sk = self.k[l][b].shape[0]
                attn[sl] = o.gqa_attention(qb, self.k[l][b].ravel(), self.v[l][b].ravel(), 1, seq, sk, c.n_q, c.n_kv,
                                           d, True).reshape(seq, -1)
            x = x + self._lin(w["o"], attn)
            h = o.rms_norm(x, gamma, c.eps)
            g, u = self._lin(w["gate"], h), self._lin(w["up"], h)
            x = x + self._lin(w["down"], o.silu(g) * u)
        hf = o.rms_norm(x, gamma, c.eps).reshape(B, seq, H)[:, -1, :]
        logits = (hf.astype(np.float32) @ self.lm_head.T).astype(np.float32)
        self.pos += seq
        nxt = np.array([o.argmax_last(logits[b]) for b in range(B)], np.int32)
        return logits, nxt
