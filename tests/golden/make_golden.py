"""Generate the golden traces in this folder by running the REFERENCE project itself.

The reference (a checkout of tenghuilee/LRQK, path given by --reference) is
imported unmodified and its ``LightAttentionIndicesFactory.prefill/.decode``
(lrqk_attention.py:1385-1613) is driven on CPU in fp32 on seeded inputs.  A few
in-process shims make the import work on this software stack; none of them
touches the arithmetic:

* four class names that newer ``transformers`` releases dropped are aliased to
  the surviving attention classes (they are only used as base classes of the
  model patches, which are not exercised here);
* ``torch.empty(..., pin_memory=True)`` has the flag dropped and
  ``torch.cuda.Stream`` is stubbed (no GPU is present);
* ``TORCHDYNAMO_DISABLE=1`` turns the ``torch.compile`` decorators into no-ops;
* the reference's compiled row-gather extension is the one built by
  ``oracle/build_ref.py`` into ``oracle/_ref/``.

The attention output is not produced by the reference on CPU (it calls a GPU
flash-attention library); it is recorded as fp32 softmax(q K^T / sqrt d) V over
the K/V rows the reference returned.

Usage:  python tests/golden/make_golden.py --reference /path/to/reference
Writes: tests/golden/<case>.npz
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

os.environ["TORCHDYNAMO_DISABLE"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

CASES = {
    # BASELINE config 0: the reference's own CPU-runnable case.
    "cfg0": dict(seed=1234, init_seed=99, bsz=1, hq=8, hkv=2, seq=4096, d=128, r=16, k=256, m=16,
                 max_iter=(2, 2), tol=1e-2, init="randn", steps=8),
    # small case that wraps the recent-token ring twice and has batch > 1; deterministic init.
    "wrap_top": dict(seed=77, init_seed=5, bsz=2, hq=4, hkv=2, seq=640, d=128, r=8, k=64, m=4,
                     max_iter=(2, 2), tol=1e-2, init="top", steps=11),
    # shared-column init, single iteration, group size 1.
    "topcol_g1": dict(seed=31, init_seed=6, bsz=1, hq=2, hkv=2, seq=512, d=128, r=16, k=32, m=8,
                      max_iter=(1, 1), tol=1e-2, init="topcol", steps=9),
    # prompt only a little longer than the resident set (k <= seq <= k + m, lrqk_attention.py:1444-1466):
    # steps 0-4 run the all-resident branch (:1526-1545), step 4 flushes the ring, steps 5.. select again.
    "short_k3": dict(seed=41, init_seed=8, bsz=2, hq=4, hkv=2, seq=67, d=128, r=8, k=64, m=8,
                     max_iter=(2, 2), tol=1e-2, init="top", steps=16),
    # prompt of exactly k rows: what DynamicLRQKCache hands over when a collected short prompt reaches
    # num_active_tokens (:1928-1958).
    "short_exact_k": dict(seed=43, init_seed=9, bsz=1, hq=4, hkv=1, seq=32, d=128, r=8, k=32, m=4,
                          max_iter=(2, 2), tol=1e-2, init="randn", steps=10),
    # weights other than 1 on all four terms: the general forms of both solvers (:218-309, :433-519).
    "weighted": dict(seed=51, init_seed=10, bsz=1, hq=4, hkv=2, seq=384, d=128, r=16, k=48, m=8,
                     max_iter=(3, 3), tol=1e-4, init="randn", steps=10, weights=(0.5, 2.0, 0.75, 1.5)),
    # only the prompt's weights differ from 1 / only the decode step's (each solver's dispatch is its own).
    "weighted_prompt_only": dict(seed=52, init_seed=11, bsz=1, hq=2, hkv=1, seq=256, d=128, r=8, k=32, m=4,
                                 max_iter=(2, 2), tol=1e-2, init="top", steps=6, weights=(1.0, 3.0, 1.0, 1.0)),
    "weighted_decode_only": dict(seed=53, init_seed=12, bsz=2, hq=2, hkv=2, seq=200, d=128, r=8, k=32, m=4,
                                 max_iter=(2, 2), tol=1e-2, init="top", steps=6, weights=(1.0, 1.0, 2.5, 0.4)),
}


def import_reference(reference_dir: str):
    import build_ref
    ext = build_ref.build_reference_ext(reference_dir)
    sys.path.insert(0, os.path.dirname(ext))
    sys.path.insert(0, reference_dir)
    from transformers.models.llama import modeling_llama
    from transformers.models.mistral import modeling_mistral
    from transformers.models.phi3 import modeling_phi3
    from transformers.models.qwen2 import modeling_qwen2
    for mod, old, new in ((modeling_qwen2, "Qwen2FlashAttention2", "Qwen2Attention"),
                          (modeling_llama, "LlamaFlashAttention2", "LlamaAttention"),
                          (modeling_mistral, "MistralFlashAttention2", "MistralAttention"),
                          (modeling_phi3, "Phi3FlashAttention2", "Phi3Attention")):
        if not hasattr(mod, old):
            setattr(mod, old, getattr(mod, new))
    if not hasattr(modeling_llama, "FlashAttentionKwargs"):
        modeling_llama.FlashAttentionKwargs = dict
    real_empty = torch.empty

    def empty_no_pin(*a, **kw):
        kw.pop("pin_memory", None)
        return real_empty(*a, **kw)

    torch.empty = empty_no_pin

    class _NoStream:
        def __init__(self, *a, **kw):
            pass

    torch.cuda.Stream = _NoStream
    import lrqk_attention as ref
    return ref


def sha(t) -> str:
    a = t.numpy() if isinstance(t, torch.Tensor) else np.asarray(t)
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def run_case(ref, name: str, c: dict) -> dict:
    import lrqk_oracle as orc
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"])
    groups = c["hq"] // c["hkv"]
    captured = {}

    class Recorder(ref.LightAttentionIndicesFactory):
        def only_indices_in_cpu(self, now_indices, new_indices):
            captured["wanted"] = new_indices.clone()
            return super().only_indices_in_cpu(now_indices, new_indices)

    f = Recorder(num_lite_tokens=c["m"], attn_topk=c["k"], num_key_value_groups=groups, r=c["r"],
                 max_iter=c["max_iter"], tol=c["tol"], capacity=c["seq"] + 64,
                 init_aq_ak_method=c["init"], weights=tuple(c.get("weights", (1.0, 1.0, 1.0, 1.0))))
    torch.manual_seed(c["init_seed"])
    f.prefill(Q.clone(), K.clone(), V.clone())
    out = {"config": np.array(json.dumps(c))}
    out["prefill_B_Q"] = f.B_Q.numpy().copy()
    out["prefill_B_K"] = f.B_K.numpy().copy()
    A_K = f.A_K
    out["prefill_A_K_every8"] = A_K[:, :, ::8].numpy().copy()
    out["prefill_A_K_sha256"] = np.array(sha(A_K))
    out["prefill_table"] = f.hit_indices[..., 0].numpy().astype(np.int32)
    out["prefill_Kres_sha256"] = np.array(sha(f.Kgpu))
    out["prefill_Vres_sha256"] = np.array(sha(f.Vgpu))
    out["host_capacity"] = np.array(f.KVcpu.data.shape[2])
    for s in range(c["steps"]):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"])
        a_len_before = len(f._A_K)
        captured.clear()
        Kres, Vres = f.decode(q.clone(), k.clone(), v.clone())
        out[f"s{s}_k_hat"] = f._A_K.data[:, :, a_len_before:a_len_before + 1].numpy().copy()
        if "wanted" in captured:        # the all-resident branch of a short prompt selects nothing
            out[f"s{s}_wanted"] = captured["wanted"][..., 0].numpy().astype(np.int32)
        out[f"s{s}_rows"] = np.array(Kres.shape[2])
        out[f"s{s}_table"] = f.hit_indices[..., 0].numpy().astype(np.int32)
        out[f"s{s}_B_Q_sha256"] = np.array(sha(f.B_Q))
        out[f"s{s}_lite"] = np.array(f.lite_indices + [f.lite_len, f.current_len, len(f.KVcpu)], dtype=np.int64)
        out[f"s{s}_Kres_sha256"] = np.array(sha(Kres))
        out[f"s{s}_Vres_sha256"] = np.array(sha(Vres))
        out[f"s{s}_attn"] = orc.attention(q, Kres, Vres).numpy().copy()
    out["final_B_Q"] = f.B_Q.numpy().copy()
    out["final_B_K"] = f.B_K.numpy().copy()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get(
        "LRQK_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")),
        help="checkout of the reference project (default: a directory \"reference\" beside this repository)")
    ap.add_argument("--cases", nargs="*", default=list(CASES))
    a = ap.parse_args()
    ref = import_reference(a.reference)
    for name in a.cases:
        data = run_case(ref, name, CASES[name])
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **data)
        print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB -> {path}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
