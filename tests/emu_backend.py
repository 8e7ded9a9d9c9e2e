"""A stand-in for the CUDA library, written with torch ops, for tests only.

It implements each kernel entry point's contract on whatever device the tensors live on, so the
host-side logic (batch building, block tables, page reuse, scheduling, trace replay) can be run on a
machine without a GPU, and so each CUDA kernel has a plain reference to be compared with on the
GPU.  It is never used by the product.
"""
import torch


class EmuBackend:
    name = "emu"

    def embed(self, ids, table, out):
        out.copy_(table[ids.long()].float())

    def rmsnorm(self, x, w, eps, out, rows):
        xr = x if rows is None else x[rows.long()]
        r = 1.0 / torch.sqrt((xr * xr).sum(-1, keepdim=True) / xr.shape[-1] + eps)
        out.copy_(((xr * r) * w.float()).to(out.dtype))

    def linear(self, a, w, bias, out, accumulate):
        y = a.float() @ w.float().T
        if bias is not None:
            y = y + bias.float()
        if accumulate:
            out.add_(y)
        else:
            out.copy_(y.to(out.dtype))

    def rope_kv_write(self, qkv, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d):
        T = qkv.shape[0]
        x = qkv.float().view(T, H + 2 * G, d)

        def rot(v):
            if n_rot == 0:
                return v
            half = n_rot // 2
            cs = cos_sin[positions.long()]
            c, s = cs[:, None, :, 0], cs[:, None, :, 1]
            a, b = v[..., :half], v[..., half:n_rot]
            return torch.cat([a * c - b * s, a * s + b * c, v[..., n_rot:]], -1)
        q_out.copy_(rot(x[:, :H]).reshape(T, H * d).to(q_out.dtype))
        if slots is None:
            return
        ok = slots >= 0
        kf, vf = k_cache.view(-1, G, d), v_cache.view(-1, G, d)
        kf[slots[ok].long()] = rot(x[:, H:H + G])[ok].to(k_cache.dtype)
        vf[slots[ok].long()] = x[:, H + G:][ok].to(v_cache.dtype)

    def paged_attention(self, q, k_cache, v_cache, meta, ctx, H, G, d, window, scale, out, tiles=None):
        T = q.shape[0]
        bs = meta.block_size
        kf, vf = k_cache.view(-1, G, d).float(), v_cache.view(-1, G, d).float()
        seqs, poss, table = ctx.token_seq.tolist(), ctx.positions.tolist(), meta.block_table.tolist()
        qf = q.float().view(T, H, d)
        res = torch.zeros(T, H, d, dtype=torch.float32, device=q.device)
        for t in range(T):
            pos, row = poss[t], table[seqs[t]]
            lo = max(0, pos - window + 1) if window > 0 else 0
            idx = []
            for j in range(lo, pos + 1):
                page = row[j // bs]
                assert page >= 0, f"token {t}: key {j} lies in an unmapped block"
                idx.append(page * bs + j % bs)
            idx = torch.tensor(idx, device=q.device)
            k, v = kf[idx], vf[idx]                       # [n, G, d]
            for h in range(H):
                g = h // (H // G)
                s = (k[:, g] @ qf[t, h]) * scale
                p = torch.softmax(s, 0)
                res[t, h] = p @ v[:, g]
        out.copy_(res.view(T, H * d).to(out.dtype))

    def swiglu(self, gu, out, interleaved):
        F = out.shape[1]
        if interleaved:
            g, u = gu[:, 0::2].float(), gu[:, 1::2].float()
        else:
            g, u = gu[:, :F].float(), gu[:, F:].float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))

    def linear_swiglu(self, a, w, gu_buf, out):
        self.linear(a, w, None, gu_buf, False)
        self.swiglu(gu_buf, out, True)

    def linear_residual_norm(self, a, w, bias, residual, norm_w, eps, xn_out):
        self.linear(a, w, bias, residual, True)
        if xn_out is not None:
            self.rmsnorm(residual, norm_w, eps, xn_out, None)

    def linear_rope_kv(self, a, w, bias, qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d):
        self.linear(a, w, bias, qkv_buf, False)
        self.rope_kv_write(qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d)

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).int())

    def error_word(self):
        return 0

    def sample(self, logits, temps, top_ks, top_ps, min_ps, uniforms, out):
        import plain_qwen2 as plain

        class Fixed:
            def __init__(self, u):
                self.u = u

            def uniform(self):
                return self.u
        rows = logits.float().cpu().numpy()
        for i in range(rows.shape[0]):
            out[i] = plain.sample(rows[i], float(temps[i]), int(top_ks[i]), float(top_ps[i]), float(min_ps[i]),
                                  Fixed(uniforms[i].cpu().numpy()))
