"""Plain-torch restatements of every kernel of the engine's kernel set, one function per
kernel, float32 arithmetic.  Two uses:
  * the `-m gpu` tests compare each CUDA kernel alone with its function here;
  * the CPU tests hand a `TorchKernels` object to the engine in place of the CUDA kernel
    set, which exercises the host logic (cache manager, step function, scheduler, replay)
    on a box without a GPU.  The engine itself has no such path.
"""
import math

import numpy as np
import torch


def ref_embed(ids, table, scale=1.0):
    return table[ids.long()].float() * scale


def ref_add_rmsnorm(residual, delta, weight, eps, rows=None, out_dtype=torch.float32):
    """Returns (new residual, normed)."""
    v = residual.float() + (delta.float() if delta is not None else 0)
    src = v if rows is None else v[rows.long()]
    y = src * torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return v, y.to(out_dtype)


def ref_rope(qkv, positions, inv_freq, heads, kv_heads, head_dim, rotary_dim):
    """Rotates the query and key heads of qkv rows; returns a new [T, (H+2Hkv)*D] float tensor."""
    T = qkv.shape[0]
    x = qkv.float().view(T, heads + 2 * kv_heads, head_dim).clone()
    if rotary_dim:
        ang = positions.float().unsqueeze(1) * inv_freq.float().unsqueeze(0)      # [T, rot/2]
        c, s = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
        half = rotary_dim // 2
        rot = x[:, :heads + kv_heads]
        x1, x2 = rot[..., :half].clone(), rot[..., half:rotary_dim].clone()
        rot[..., :half] = x1 * c - x2 * s
        rot[..., half:rotary_dim] = x2 * c + x1 * s
    return x.view(T, -1)


def ref_store(cache_layer, rotated, slots, heads, kv_heads, head_dim):
    """cache_layer [pages, 2, Hkv, page, D]; writes k and v rows of `rotated` at `slots`."""
    T = rotated.shape[0]
    page_size = cache_layer.shape[3]
    x = rotated.view(T, heads + 2 * kv_heads, head_dim)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        p, o = divmod(s, page_size)
        cache_layer[p, 0, :, o, :] = x[t, heads:heads + kv_heads].to(cache_layer.dtype)
        cache_layer[p, 1, :, o, :] = x[t, heads + kv_heads:].to(cache_layer.dtype)


def ref_paged_attention(q, cache_layer, block_table, token_request, positions, heads, kv_heads, head_dim,
                        window=0, scale=0.0):
    """q [T, >= heads*head_dim] (query heads first); returns [T, heads*head_dim] float32."""
    T = q.shape[0]
    page_size = cache_layer.shape[3]
    scale = scale or 1.0 / math.sqrt(head_dim)
    group = heads // kv_heads
    out = torch.zeros(T, heads, head_dim, dtype=torch.float32, device=q.device)
    for t in range(T):
        pos = int(positions[t])
        lo = max(0, pos - window + 1) if window > 0 else 0
        table = block_table[int(token_request[t])]
        idx = torch.arange(lo, pos + 1, device=q.device)
        pages = table[(idx // page_size).long()].long()
        offs = (idx % page_size).long()
        k = cache_layer[pages, 0, :, offs, :].float()        # [n, Hkv, D]
        v = cache_layer[pages, 1, :, offs, :].float()
        qt = q[t, :heads * head_dim].float().view(heads, head_dim)
        kk = k.repeat_interleave(group, dim=1)                # [n, H, D]
        vv = v.repeat_interleave(group, dim=1)
        sc = torch.einsum("hd,nhd->hn", qt, kk) * scale
        p = torch.softmax(sc, dim=-1)
        out[t] = torch.einsum("hn,nhd->hd", p, vv)
    return out.view(T, heads * head_dim)


def ref_linear(x, weight, swiglu=False):
    y = x.float() @ weight.float().t()
    if swiglu:
        n = weight.shape[0] // 2
        return torch.nn.functional.silu(y[:, :n]) * y[:, n:]
    return y


def ref_silu_mul(gu):
    n = gu.shape[1] // 2
    g = gu.float()
    return torch.nn.functional.silu(g[:, :n]) * g[:, n:]


_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix64(z):
    z = z.astype(np.uint64)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def ref_gumbel(key, vocab):
    """The kernel's noise for one row: key is the row's 64-bit key as a Python int (unsigned)."""
    with np.errstate(over="ignore"):
        i = np.arange(1, vocab + 1, dtype=np.uint64)
        r = _mix64(np.uint64(key) + np.uint64(0x9E3779B97F4A7C15) * i)
    u = ((r >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return torch.from_numpy(-np.log(-np.log(u)).astype(np.float32))


def ref_sample(logits, temperature=None, keys=None):
    """Returns (ids, perturbed rows) -- perturbed rows let a test skip near-ties."""
    rows = []
    for r in range(logits.shape[0]):
        row = logits[r].float().cpu()
        T = float(temperature[r]) if temperature is not None else 0.0
        if T > 0:
            key = int(keys[r]) & 0xFFFFFFFFFFFFFFFF
            row = row / T + ref_gumbel(key, row.shape[0])
        rows.append(row)
    rows = torch.stack(rows)
    return rows.argmax(-1).to(torch.int32), rows


class TorchKernels:
    """Same method names and argument order as iitj_llm_coopt_b200.kernels.Kernels."""

    launches = 0

    def embed(self, ids, table, out, scale=1.0):
        out.copy_(ref_embed(ids, table, scale))
        return out

    def add_rmsnorm(self, residual, delta, weight, eps, out, rows=None):
        v, y = ref_add_rmsnorm(residual, delta, weight, eps, rows, out.dtype)
        if rows is None and delta is not None:
            residual.copy_(v)
        out.copy_(y)
        return out

    def rope_tables(self, positions, inv_freq, cos, sin):
        ang = positions.float().unsqueeze(1) * inv_freq.float().unsqueeze(0)
        cos.copy_(ang.cos())
        sin.copy_(ang.sin())
        return cos, sin

    def rope_store(self, qkv, positions, inv_freq, slots, cache_layer, heads, kv_heads, head_dim, rotary_dim, tables=None):
        rot = ref_rope(qkv, positions, inv_freq, heads, kv_heads, head_dim, rotary_dim).to(qkv.dtype)
        if slots is not None:
            ref_store(cache_layer, rot, slots, heads, kv_heads, head_dim)
        qkv[:, :heads * head_dim] = rot[:, :heads * head_dim]
        return qkv

    def silu_mul(self, gu, act):
        act.copy_(ref_silu_mul(gu))
        return act

    def attention(self, qkv, cache_layer, meta, out, heads, kv_heads, head_dim, window=0, scale=0.0):
        out.copy_(ref_paged_attention(qkv, cache_layer, meta.block_table, meta.token_request, meta.positions,
                                      heads, kv_heads, head_dim, window, scale))
        return out

    def linear(self, x, weight, out, swiglu=False, defer=False):
        out.copy_(ref_linear(x, weight, swiglu))     # never split: `defer` has nothing to leave for later
        return out

    health_codes = (0, 0, 0, 0)     # what `sample` reports as the library's health words (tests set a failure here)

    def scale_(self, x, scale):
        return x.mul_(scale)

    def sample(self, logits, temperature, keys, out, health=None):
        ids, _ = ref_sample(logits, temperature, keys)
        out.copy_(ids)
        if health is not None:
            health[:4] = torch.tensor(self.health_codes, dtype=torch.int32)
        return out

    def check_health(self, codes=None):
        codes = list(self.health_codes if codes is None else codes)
        if any(codes):
            self.health_codes = (0, 0, 0, 0)
            raise RuntimeError(f"a kernel gave up: {codes}")
