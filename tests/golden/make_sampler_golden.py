"""Makes tests/golden/sampler_reference_processing.json: what the reference's own
``Sampler.process`` (ErnestW2019/acorninfer, acorninfer/sampler.py:38-56, imported on the CPU) leaves of seeded
logits for a dozen (temperature, top-k, top-p) settings, so that the plain ``process_logits`` under
tests/plain/ can be checked against the reference without the reference being present.

Run from the repository root with the reference on the path:

    PYTHONPATH=<path to the acorninfer checkout> python tests/golden/make_sampler_golden.py

The input logits are stored with the outputs (float32 values written as decimal strings by
``repr``, which round-trips), so the check does not depend on a random generator.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
CASES = [(1.0, 0, 1.0), (0.7, 0, 1.0), (2.5, 0, 1.0), (1.0, 1, 1.0), (1.0, 5, 1.0), (0.8, 40, 1.0), (1.0, 500, 1.0),
         (1.0, 0, 0.9), (0.6, 0, 0.5), (1.3, 0, 0.05), (0.7, 20, 0.95), (1.1, 7, 0.6), (0.9, 3, 0.999)]
VOCAB = 211


def main() -> None:
    from acorninfer.sampler import Sampler, SamplingParams

    g = torch.Generator().manual_seed(5)
    out = []
    for n, (temperature, top_k, top_p) in enumerate(CASES):
        logits = 3.0 * torch.randn(VOCAB, generator=g)
        if n % 3 == 0:
            logits[10:14] = logits[10]            # exact ties, also at the thresholds
        processed = Sampler(SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p)).process(logits.clone())
        kept = torch.isfinite(processed)
        out.append({"temperature": temperature, "top_k": top_k, "top_p": top_p,
                    "logits": [repr(float(x)) for x in logits],
                    "kept": [int(i) for i in kept.nonzero().flatten()],
                    "processed_kept": [repr(float(x)) for x in processed[kept]]})
    (HERE / "sampler_reference_processing.json").write_text(json.dumps(out) + "\n")
    print("wrote", HERE / "sampler_reference_processing.json", "with", len(out), "cases")


if __name__ == "__main__":
    main()
