"""Generates the committed golden fixtures by running the UNMODIFIED reference build
(oracle/_ref/_C.so, made by `make -C oracle ref`) on its paras:0 host engine, in a child
process (oracle/ref_run.py).  Run from the repository root, where the reference sources
are mounted:

    python tests/golden/make_golden.py

Each fixture is a small torch.save'd dict {"op", "args", "out"}; inputs are seeded draws
with the shapes of the benchmark configurations scaled down so that every file stays in
the tens of kilobytes.  tests/test_oracle_pins.py holds the oracle restatement to them
bit-for-bit; the GPU parity tests hold the CUDA kernels to them within tolerance.
"""
import os
import subprocess
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def cases():
    g = torch.Generator().manual_seed(20261125)

    def R(*shape, dt=torch.float32, mean=0.0, std=1.0):
        return (mean + std * torch.randn(*shape, generator=g)).to(dt)

    out = []
    for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        # config 1 shape family: B2 H4 S128 D64 causal (shrunk to S=48) + the reference tests' own shape
        q, k, v = R(2, 4, 48, 64, dt=dt), R(2, 4, 48, 64, dt=dt), R(2, 4, 48, 64, dt=dt)
        out.append((f"sdpa_causal_d64_{tag}", "sdpa", {"q": q, "k": k, "v": v, "is_causal": True}))
        q, k, v = R(2, 4, 8, 16, dt=dt), R(2, 4, 8, 16, dt=dt), R(2, 4, 8, 16, dt=dt)
        out.append((f"sdpa_basic_{tag}", "sdpa", {"q": q, "k": k, "v": v}))
        # Lq != Lk causal: pins the top-left alignment of the mask
        q, k, v = R(1, 2, 20, 128, dt=dt), R(1, 2, 40, 128, dt=dt), R(1, 2, 40, 128, dt=dt)
        out.append((f"sdpa_causal_lq20_lk40_{tag}", "sdpa", {"q": q, "k": k, "v": v, "is_causal": True}))
        # GQA 8 query heads over 2 kv heads, D=128, ragged length (not a multiple of any tile)
        q, k, v = R(1, 8, 70, 128, dt=dt), R(1, 2, 70, 128, dt=dt), R(1, 2, 70, 128, dt=dt)
        out.append((f"sdpa_causal_gqa_{tag}", "sdpa",
                    {"q": q, "k": k, "v": v, "is_causal": True, "enable_gqa": True}))
        # decode step: q_len 1 over a longer cache, non-causal, GQA 4:1
        q, k, v = R(2, 8, 1, 128, dt=dt), R(2, 2, 300, 128, dt=dt), R(2, 2, 300, 128, dt=dt)
        out.append((f"sdpa_decode_gqa_{tag}", "sdpa", {"q": q, "k": k, "v": v, "enable_gqa": True}))
        # explicit scale
        q, k, v = R(1, 2, 16, 32, dt=dt), R(1, 2, 16, 32, dt=dt), R(1, 2, 16, 32, dt=dt)
        out.append((f"sdpa_scale_{tag}", "sdpa", {"q": q, "k": k, "v": v, "scale": 0.17}))
        # masks
        mask = torch.rand(1, 2, 16, 16, generator=g) > 0.3
        mask[..., 0] = True
        out.append((f"sdpa_boolmask_{tag}", "sdpa", {"q": q, "k": k, "v": v, "attn_mask": mask}))
        bias = (0.1 * torch.randn(1, 2, 16, 16, generator=g)).to(dt)
        out.append((f"sdpa_addmask_{tag}", "sdpa", {"q": q, "k": k, "v": v, "attn_mask": bias}))

        x = R(24, 256, dt=dt)
        w = R(256, dt=dt, mean=1.0, std=0.1)
        out.append((f"rmsnorm_aten_{tag}", "rms_norm_aten",
                    {"x": x, "weight": w, "normalized_shape": [256], "eps": 1e-6}))
        out.append((f"rmsnorm_aten_noweight_{tag}", "rms_norm_aten",
                    {"x": x, "weight": None, "normalized_shape": [256], "eps": None}))
        x3 = R(3, 4, 5, dt=dt)
        out.append((f"rmsnorm_aten_multidim_{tag}", "rms_norm_aten",
                    {"x": x3, "weight": None, "normalized_shape": [4, 5], "eps": 1e-5}))
        out.append((f"rmsnorm_paras_{tag}", "rms_norm_paras", {"x": x, "weight": w, "eps": 1e-6}))
        xo = R(5, 100, dt=dt)  # odd width: not a multiple of the vector size
        wo = R(100, dt=dt, mean=1.0, std=0.1)
        out.append((f"rmsnorm_paras_odd_{tag}", "rms_norm_paras", {"x": xo, "weight": wo, "eps": 1e-6}))
        go = R(24, 256, dt=dt)
        rstd = 1.0 / torch.sqrt((x.double() ** 2).mean(-1) + 1e-6)
        out.append((f"rmsnorm_paras_bwd_{tag}", "rms_norm_paras_backward",
                    {"grad_out": go, "x": x, "weight": w, "rstd": rstd.float()}))

        gate, up = R(17, 77, dt=dt), R(17, 77, dt=dt)
        out.append((f"swiglu_paras_{tag}", "swiglu_paras", {"gate": gate, "up": up}))
        out.append((f"swiglu_composite_{tag}", "swiglu_composite", {"x": up, "gate": gate}))
        out.append((f"swiglu_paras_bwd_{tag}", "swiglu_paras_backward",
                    {"grad_out": R(17, 77, dt=dt), "gate": gate, "up": up}))
        xr = R(6, 32, dt=dt)
        out.append((f"rotate_half_{tag}", "rotate_half", {"x": xr}))
        out.append((f"rotate_half_bwd_{tag}", "rotate_half_backward", {"grad_out": xr}))
    return out


def grad_cases():
    """Attention gradients of the reference (autograd through its composite).  A generator of their
    own, so that adding cases here leaves the draws of cases() unchanged."""
    g = torch.Generator().manual_seed(20261126)

    def R(*shape, dt=torch.float32):
        return torch.randn(*shape, generator=g).to(dt)

    # 3-D (batch, seq, dim) inputs: the reference differentiates those; with 4-D inputs its own
    # backward of the batched product fails ("BmmBackward0 returned an invalid gradient ... got
    # [2, 200, 200] but expected shape compatible with [1, 2, 200, 200]"), so there is nothing to pin
    out = []
    for dt, tag in ((torch.bfloat16, "bf16"),):   # the gradient kernels take 16-bit tensors only
        # two query tiles over two key tiles, causal: the diagonal tiles and an off-diagonal one
        q, k, v, d = R(1, 200, 128, dt=dt), R(1, 200, 128, dt=dt), R(1, 200, 128, dt=dt), R(1, 200, 128, dt=dt)
        out.append((f"sdpa_grad_causal_{tag}", "sdpa_grad", {"q": q, "k": k, "v": v, "dout": d, "is_causal": True}))
        # full attention, Lq != Lk, head dim 64
        q, k, v, d = R(2, 72, 64, dt=dt), R(2, 136, 64, dt=dt), R(2, 136, 64, dt=dt), R(2, 72, 64, dt=dt)
        out.append((f"sdpa_grad_full_d64_{tag}", "sdpa_grad", {"q": q, "k": k, "v": v, "dout": d}))
    return out


def dropout_cases():
    """The math op's two results (output, weights after dropout) with the reference's own dropout:
    its Philox stream re-seeded per case, and a caller's dropout_mask."""
    g = torch.Generator().manual_seed(20261127)

    def R(*shape, dt=torch.float32):
        return torch.randn(*shape, generator=g).to(dt)

    out = []
    for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        q, k, v = R(1, 4, 24, 16, dt=dt), R(1, 2, 40, 16, dt=dt), R(1, 2, 40, 16, dt=dt)
        out.append((f"sdpa_math_dropout_{tag}", "sdpa_math",
                    {"q": q, "k": k, "v": v, "dropout_p": 0.25, "seed": 1234, "enable_gqa": True}))
        out.append((f"sdpa_math_weights_causal_{tag}", "sdpa_math",
                    {"q": q, "k": k, "v": v, "is_causal": True, "enable_gqa": True}))
        dm = (torch.rand(1, 4, 24, 40, generator=g) > 0.5).to(dt)
        out.append((f"sdpa_math_dropout_mask_{tag}", "sdpa_math",
                    {"q": q, "k": k, "v": v, "dropout_p": 0.3, "dropout_mask": dm, "enable_gqa": True}))
    return out


def rope_cases():
    """Rotary embedding as a user of the reference composes it (x * cos + rotate_half(x) * sin with the
    reference's mul, add and paras::rotate_half) in front of its attention."""
    g = torch.Generator().manual_seed(20261128)

    def R(*shape, dt=torch.float32):
        return torch.randn(*shape, generator=g).to(dt)

    def tables(rows, D, dt):
        inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        ang = torch.arange(rows, dtype=torch.float64)[:, None] * inv[None, :]
        emb = torch.cat((ang, ang), dim=-1)
        return emb.cos().to(dt), emb.sin().to(dt)

    out = []
    for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        # causal GQA, then a decode step at position 29 of a 30-key cache (small head dim: the
        # rounding of the three element-wise steps is what is being pinned)
        cos, sin = tables(30, 32, dt)
        q, k, v = R(1, 2, 24, 32, dt=dt), R(1, 1, 24, 32, dt=dt), R(1, 1, 24, 32, dt=dt)
        out.append((f"rope_sdpa_causal_gqa_{tag}", "rope_sdpa",
                    {"q": q, "k": k, "v": v, "cos": cos, "sin": sin, "is_causal": True, "enable_gqa": True}))
        q, k, v = R(2, 2, 1, 32, dt=dt), R(2, 1, 30, 32, dt=dt), R(2, 1, 30, 32, dt=dt)
        out.append((f"rope_sdpa_decode_{tag}", "rope_sdpa",
                    {"q": q, "k": k, "v": v, "cos": cos, "sin": sin, "q_pos0": 29, "enable_gqa": True}))
    # head dim 128 (the shape the attention kernel rotates in its prologue), 16 bit
    cos, sin = tables(40, 128, torch.bfloat16)
    q, k, v = R(1, 2, 40, 128, dt=torch.bfloat16), R(1, 1, 40, 128, dt=torch.bfloat16), R(1, 1, 40, 128, dt=torch.bfloat16)
    out.append(("rope_sdpa_causal_d128_bf16", "rope_sdpa",
                {"q": q, "k": k, "v": v, "cos": cos, "sin": sin, "is_causal": True, "enable_gqa": True}))
    return out


def main():
    if "--rope" in sys.argv:     # only the rotary-embedding fixtures
        globals()["cases"] = rope_cases
    if "--dropout" in sys.argv:  # only the dropout / weights fixtures
        globals()["cases"] = dropout_cases
    if "--grad" in sys.argv:     # only the gradient fixtures
        globals()["cases"] = grad_cases
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_loader
    if not ref_loader.available():
        raise SystemExit("oracle/_ref/_C.so missing: run `make -C oracle ref` first")
    cs = cases()
    jobs = [{"op": op, "args": args} for _, op, args in cs]
    with tempfile.TemporaryDirectory() as td:
        torch.save(jobs, os.path.join(td, "jobs.pt"))
        subprocess.check_call([sys.executable, os.path.join(ROOT, "oracle", "ref_run.py"),
                               os.path.join(td, "jobs.pt"), os.path.join(td, "res.pt")])
        res = torch.load(os.path.join(td, "res.pt"))
    total = 0
    for (name, op, args), r in zip(cs, res):
        path = os.path.join(HERE, name + ".pt")
        torch.save({"op": op, "args": args, "out": r["out"]}, path)
        total += os.path.getsize(path)
    print(f"wrote {len(cs)} fixtures, {total / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
