"""Trace replay: feed given token ids through a model step by step and write logits.

Nothing is sampled.  The replayer drives the same model object, step function, cache and
kernels that generation uses.  The closest things in the reference are its debug forward-pass
command over explicit ids (src/DotLLM.Cli/Commands/Debug/DebugForwardPassCommand.cs:93-99,140-226)
and the forced-token stepping of its CPU/GPU comparison test
(tests/DotLLM.Tests.Unit/Cuda/CudaLogitComparisonTest.cs:57-89).

Input: one JSON object per line,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` give each request's next tokens and the offsets among them whose logits are wanted;
an id seen for the first time opens a sequence.  ``end`` lists requests that are finished after
the step; their slots and pages are given back.  For a step that wants anything, the logits are
written to ``<out>/<step>.f32`` as little-endian float32 [wanted, vocab], in the order of the
entries and of ``want``.  After every step ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

from ..errors import StepError
from .step import StepEntry


class TraceReplayer:
    def __init__(self, model, max_tokens, out_dir):
        self.model = model
        self.cache = model.new_cache(max_tokens)
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.sequences = {}

    @staticmethod
    def check_kernels():
        """Raise if a kernel gave up on a bounded wait (its result would be wrong)."""
        from ..kernels import library
        library.check_status()

    def run_step(self, record):
        step_id = record["step"]
        entries = []
        opened = []
        try:
            for e in record.get("entries", []):
                rid = e["id"]
                if rid not in self.sequences:
                    self.sequences[rid] = self.cache.open_sequence()
                    opened.append(rid)
                entries.append(StepEntry(self.sequences[rid], list(e["tokens"]), list(e.get("want", []))))
            if entries:
                logits = self.model.step(self.cache, entries)
                if logits.shape[0] > 0:
                    data = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                    data.tofile(self.out_dir / f"{step_id}.f32")
                    self.check_kernels()
        except Exception:
            for rid in opened:                      # a refused step leaves no half-opened request
                self.cache.close_sequence(self.sequences.pop(rid))
            raise
        for rid in record.get("end", []):
            if rid not in self.sequences:
                raise StepError(f"step {step_id}: cannot end unknown request {rid!r}")
            self.cache.close_sequence(self.sequences.pop(rid))
        return step_id

    def run(self, lines, out=sys.stdout):
        for line in lines:
            line = line.strip()
            if not line:
                continue
            step_id = self.run_step(json.loads(line))
            out.write(f"done {step_id}\n")
            out.flush()


def main(argv=None):
    import argparse
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--device", default="cuda")
    args = parser.parse_args(argv)
    from ..model import Model
    model = Model.load(args.model, dtype=args.dtype, device=args.device)
    TraceReplayer(model, args.max_tokens, args.out).run(sys.stdin)
    return 0
