"""Child-process runner for the UNMODIFIED reference build on its ``paras:0`` host engine.

TEST INFRASTRUCTURE ONLY (checker and CPU-baseline timer); never on the product path.

    python oracle/ref_run.py jobs.pt results.pt

``jobs.pt`` is a ``torch.save``'d list of dicts ``{"op": name, "args": {...}, "repeat": n}``;
``results.pt`` receives a list of ``{"out": tensor | tuple, "seconds": best wall time,
"threads": host threads the reference engine used}``.  Ops go through exactly the public
entry points a user of the reference calls (F.scaled_dot_product_attention,
torch.ops.aten.rms_norm, torch.ops.paras.*, torch.ops.torch_paras.swiglu).
"""
import os
import sys
import time

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import ref_loader  # noqa: E402

DEV = "paras:0"
_MOD = None   # the reference's extension module, set by main()


def _dev(t):
    return t.to(DEV) if torch.is_tensor(t) else t


def _cpu(o):
    if torch.is_tensor(o):
        return o.cpu()
    if isinstance(o, (tuple, list)):
        return tuple(_cpu(x) for x in o)
    return o


def run_op(op, a):
    if op == "sdpa":
        q, k, v = _dev(a["q"]), _dev(a["k"]), _dev(a["v"])
        mask = _dev(a.get("attn_mask"))
        kw = {}
        if a.get("scale") is not None:
            kw["scale"] = a["scale"]
        if a.get("enable_gqa"):
            kw["enable_gqa"] = True
        return lambda: F.scaled_dot_product_attention(
            q, k, v, attn_mask=mask, is_causal=bool(a.get("is_causal", False)), **kw)
    if op == "sdpa_math":
        # the math op with its two results (output, weights after dropout); the device's generator is
        # re-seeded first, so the dropout draws counters (seed, sequence 0)
        q, k, v = _dev(a["q"]), _dev(a["k"]), _dev(a["v"])
        mask, dmask = _dev(a.get("attn_mask")), _dev(a.get("dropout_mask"))

        def run_math():
            _MOD.manual_seed_all(int(a.get("seed", 0)))
            return torch.ops.aten._scaled_dot_product_attention_math(
                q, k, v, mask, float(a.get("dropout_p", 0.0)), bool(a.get("is_causal", False)), dmask,
                scale=a.get("scale"), enable_gqa=bool(a.get("enable_gqa", False)))
        return run_math
    if op == "sdpa_grad":
        # gradients by autograd through the reference's composite attention (attention_ops.cpp:71-136
        # and the backward kernels its operators register, e.g. softmax backward, pointwise_ops.cpp:
        # 994-1062): returns (out, dq, dk, dv)
        kw = {"enable_gqa": True} if a.get("enable_gqa") else {}

        def run():
            q, k, v = (_dev(a[n]).detach().requires_grad_(True) for n in ("q", "k", "v"))
            out = F.scaled_dot_product_attention(q, k, v, is_causal=bool(a.get("is_causal", False)), **kw)
            out.backward(_dev(a["dout"]))
            return out.detach(), q.grad, k.grad, v.grad
        return run
    if op == "rms_norm_aten":
        x, w = _dev(a["x"]), _dev(a.get("weight"))
        return lambda: torch.ops.aten.rms_norm(x, list(a["normalized_shape"]), w, a.get("eps"))
    if op == "rms_norm_paras":
        x, w = _dev(a["x"]), _dev(a["weight"])
        return lambda: torch.ops.paras.rms_norm(x, w, float(a["eps"]))
    if op == "rms_norm_paras_backward":
        g, x, w, r = _dev(a["grad_out"]), _dev(a["x"]), _dev(a["weight"]), _dev(a["rstd"])
        return lambda: torch.ops.paras.rms_norm_backward(g, x, w, r)
    if op == "swiglu_paras":
        g, u = _dev(a["gate"]), _dev(a["up"])
        return lambda: torch.ops.paras.swiglu(g, u)
    if op == "swiglu_paras_backward":
        d, g, u = _dev(a["grad_out"]), _dev(a["gate"]), _dev(a["up"])
        return lambda: torch.ops.paras.swiglu_backward(d, g, u)
    if op == "swiglu_composite":
        x, g = _dev(a["x"]), _dev(a["gate"])
        return lambda: torch.ops.torch_paras.swiglu(x, g)
    if op == "rotate_half":
        x = _dev(a["x"])
        return lambda: torch.ops.paras.rotate_half(x)
    if op == "rope_sdpa":
        # rotary embedding composed from the reference's own operators (mul.out, add.out,
        # paras::rotate_half), then its attention: returns (rotated q, rotated k, attention output)
        q, k, v = _dev(a["q"]), _dev(a["k"]), _dev(a["v"])
        cos, sin = _dev(a["cos"]), _dev(a["sin"])
        pos0 = int(a.get("q_pos0", 0))
        kw = {"enable_gqa": True} if a.get("enable_gqa") else {}

        def run_rope():
            cq, sq = cos[pos0:pos0 + q.shape[-2]], sin[pos0:pos0 + q.shape[-2]]
            ck, sk = cos[:k.shape[-2]], sin[:k.shape[-2]]
            qr = q * cq + torch.ops.paras.rotate_half(q) * sq
            kr = k * ck + torch.ops.paras.rotate_half(k) * sk
            out = F.scaled_dot_product_attention(qr, kr, v, is_causal=bool(a.get("is_causal", False)), **kw)
            return qr, kr, out
        return run_rope
    if op == "rotate_half_backward":
        x = _dev(a["grad_out"])
        return lambda: torch.ops.paras.rotate_half_backward(x)
    raise ValueError(f"unknown op {op}")


def main():
    jobs_path, out_path = sys.argv[1], sys.argv[2]
    # The reference's host engine runs on torch.get_num_threads() threads (host_thread_count,
    # csrc/compat/paras_compat.cpp:70-82).  A launcher may have exported OMP_NUM_THREADS=1 to
    # this process; PARAS_REF_THREADS states the count the caller wants instead.
    if os.environ.get("PARAS_REF_THREADS"):
        torch.set_num_threads(int(os.environ["PARAS_REF_THREADS"]))
    global _MOD
    mod = _MOD = ref_loader.load()
    jobs = torch.load(jobs_path)
    results = []
    for job in jobs:
        fn = run_op(job["op"], job["args"])
        best, out = None, None
        for _ in range(max(1, int(job.get("repeat", 1)))):
            t0 = time.perf_counter()
            out = fn()
            mod.synchronize_all()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        results.append({"out": _cpu(out) if job.get("keep_out", True) else None,
                        "seconds": best, "threads": torch.get_num_threads()})
    torch.save(results, out_path)


if __name__ == "__main__":
    main()
