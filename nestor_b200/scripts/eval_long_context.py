"""Per-position cross-entropy of a checkpoint on long held-out documents.

The context length and RoPE base are exported (``DCLM_BLOCK_SIZE`` / ``DCLM_ROPE_BASE``) before the
registry builds the model, as they are read when the experiment function runs. One backbone pass per
document, the head applied in chunks (reference ``scripts/eval_long_context.py:59-64``,
``nestor/eval/long_context.py:75-117``).
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--experiment", required=True); ap.add_argument("--checkpoint", type=Path, required=True)
    ap.add_argument("--data", type=Path, required=True); ap.add_argument("--seq-len", type=int, required=True)
    ap.add_argument("--rope-base", type=float, default=None); ap.add_argument("--documents", type=int, default=200)
    ap.add_argument("--head-chunk", type=int, default=4096); ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--output", type=Path, default=None)
    a = ap.parse_args(argv)
    os.environ["DCLM_BLOCK_SIZE"] = str(a.seq_len)
    if a.rope_base is not None:
        os.environ["DCLM_ROPE_BASE"] = str(a.rope_base)
    from nestor_b200.data.documents import document_spans, load_document, open_token_bin, select_documents
    from nestor_b200.eval.loading import load_experiment_checkpoint
    from nestor_b200.eval.long_context import PerPositionLoss, sequence_nll

    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model, info = load_experiment_checkpoint(a.experiment, a.checkpoint, device=device,
                                             dtype=torch.bfloat16 if a.bf16 else torch.float32)
    tokens, eot = open_token_bin(a.data)
    spans = select_documents(document_spans(tokens, eot), min_tokens=a.seq_len, max_docs=a.documents)
    acc = PerPositionLoss(a.seq_len)
    for span in spans:
        doc = torch.from_numpy(load_document(tokens, span, max_tokens=a.seq_len)).unsqueeze(0).to(device)
        nll, _ = sequence_nll(model, doc, head_chunk=a.head_chunk)
        acc.add(nll, start=1)
    res = {**acc.to_dict(), **info, "documents": int(len(spans)), "seq_len": a.seq_len}
    print(json.dumps({k: v for k, v in res.items() if k not in ("mean_by_position", "moving_average")}, indent=2))
    if a.output:
        a.output.write_text(json.dumps(res))


if __name__ == "__main__":
    main()
