"""Teacher-forced baseline probes from the `transformers` implementation of a checkpoint.

The independent side of a quality comparison: the source checkpoint is run with the library's
own model code (no kernel, codec or engine of this repository), and the probe records it
writes are paired with those of the converted model (``orinfer score-model --jsonl ...
--query-from``) by ``orinfer bench quality``.  Same role as the reference's
tools/eval/reference_bf16.py (an independent full-sequence teacher-forced prefill; not a
timing tool).

    python -m orinfer_b200.bench.hf_reference HF_DIR --tokens 1,2,3,4 --jsonl base.jsonl
"""

from __future__ import annotations

import argparse
import json

import torch

from . import quality as Q


def probes(model_dir: str, tokens, case_id: str = "case", dtype: str = "float32",
           device: str = "cpu"):
    from transformers import AutoModelForCausalLM
    model = AutoModelForCausalLM.from_pretrained(model_dir, dtype=getattr(torch, dtype))
    model = model.to(device).eval()
    ids = torch.tensor([list(tokens)], device=device)
    with torch.no_grad():
        logits = model(ids).logits[0].float().cpu().numpy()
    return Q.probes_from_logits(logits, list(tokens), case_id, "prefill")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("model_dir")
    ap.add_argument("--tokens", required=True, help="comma-separated token ids")
    ap.add_argument("--jsonl", required=True)
    ap.add_argument("--case-id", default="case")
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16", "float16"])
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    out = probes(a.model_dir, [int(x) for x in a.tokens.split(",")], a.case_id, a.dtype, a.device)
    Q.write_jsonl(a.jsonl, out)
    print(json.dumps({"probes": len(out), "file": a.jsonl}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
