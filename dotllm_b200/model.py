"""The Python entry point: load a model folder (or random weights), step it, generate with it.

Mirrors the reference's top-level objects: ``ModelLoader`` (src/DotLLM.Models/ModelLoader.cs:21-28),
``IModel`` with ``Config`` and ``Forward`` (src/DotLLM.Core/Models/IModel.cs:9-35) and
``TextGenerator`` (src/DotLLM.Engine/TextGenerator.cs:68).  The model class is chosen by
config.json through the architecture registry.
"""
from __future__ import annotations

import torch

from .config.registry import build_spec, load_config
from .engine.decode_graph import DecodeGraphs, StepGraphs
from .engine.generate import TextGenerator
from .engine.step import StepEntry, run_step
from .errors import ConfigError, KernelError
from .models.decoder import DecoderModel
from .parts.base import Runtime
from .sampling.options import InferenceOptions
from .sampling.pipeline import sample_rows
from .weights.loader import load_into
from .weights.random_init import init_random

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


class _IdFetcher:
    """Brings a step's sampled ids to the host together with the kernels' status word: one small
    device-to-host copy into pinned memory and one wait per step (no device-wide synchronisation,
    no second read for the status)."""

    def __init__(self, device):
        self.device = device
        self.pinned = torch.empty(4096, dtype=torch.int32).pin_memory()

    def start(self, ids):
        """Send the copy; what follows on the stream (the next step, started ahead) does not delay it."""
        from .kernels import library
        n = ids.numel()
        if n + 1 > self.pinned.numel():
            self.pinned = torch.empty(2 * (n + 1), dtype=torch.int32).pin_memory()
        both = torch.cat([ids.to(torch.int32).reshape(-1), library.status_word(self.device)])
        self.pinned[:n + 1].copy_(both, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return n, done

    def finish(self, pending):
        from .kernels import library
        n, done = pending
        done.synchronize()
        values = self.pinned[:n + 1].tolist()
        if values[n]:
            library.check_status()                           # raises with the kernel's reason and clears the word
        return values[:n]

    def __call__(self, ids):
        return self.finish(self.start(ids))


class _EventClock:
    """Marks are CUDA events on the current stream; their distances are read when the batch is over."""

    def mark(self):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    @staticmethod
    def ms(a, b):
        b.synchronize()
        return a.elapsed_time(b)


def parse_dtype(dtype):
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ConfigError(f"models run in bfloat16 or float32, not {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ConfigError(f"unknown dtype {dtype!r}; use 'bfloat16' or 'float32'") from None


def parse_device(device):
    """'cuda', 'cuda:N', or the reference's 'gpu' / 'gpu:N' (src/DotLLM.Cli/Commands/RunCommand.cs:95-98)."""
    if isinstance(device, torch.device):
        return device
    name = str(device).lower().replace("gpu", "cuda")
    dev = torch.device(name)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
    return dev


class Model:
    """A loaded model: its typed configuration, its description, its parts on the device."""

    def __init__(self, config, spec, decoder):
        self.config = config
        self.spec = spec
        self.decoder = decoder
        self.runtime = decoder.runtime
        self._generator = None

    # ---------------------------------------------------------------- making
    @classmethod
    def _skeleton(cls, config, dtype, device, spec=None):
        runtime = Runtime(parse_dtype(dtype), parse_device(device))
        if runtime.device.type != "cuda":
            raise KernelError(f"models run on a CUDA device (sm_100a); got device {runtime.device}")
        torch.cuda.set_device(runtime.device)
        spec = spec or build_spec(config)
        return cls(config, spec, DecoderModel(spec, runtime))

    @classmethod
    def load(cls, folder, dtype="bfloat16", device="cuda"):
        """From a folder with config.json and model.safetensors (or an index and shards)."""
        config = load_config(folder)
        model = cls._skeleton(config, dtype, device)
        load_into(model.decoder, folder)
        return model

    @classmethod
    def random(cls, config, seed=0, dtype="bfloat16", device="cuda", on_device=False, spec=None):
        """Random weights drawn in memory from (config, seed); nothing is written.  The numbers are those
        that ``write_random_model(folder, config, seed)`` stores, so a model made here and one loaded
        from such a folder are the same model.  ``on_device=True`` draws with the device's generator
        instead: another stream of numbers, seconds instead of minutes for a model of many gigabytes."""
        model = cls._skeleton(config, dtype, device, spec)
        init_random(model.decoder, seed, on_device=on_device)
        return model

    # --------------------------------------------------------------- running
    def new_cache(self, max_tokens, max_sequences=None):
        return self.decoder.new_cache(max_tokens, max_sequences)

    def step(self, cache, entries, graphs=False):
        """Run one step; ``entries`` are StepEntry objects (or (sequence, tokens[, want]) tuples).
        Returns float32 logits [wanted, vocab].

        With ``graphs`` a step that brings one token per sequence and wants each one's logits is
        replayed as a CUDA graph (captured once per batch size), and any other step is replayed from a
        graph of its exact shape once that shape has been seen twice (prompts of equal lengths, chunks
        of a fixed size); the returned tensor is then a buffer that the next such step overwrites.
        A model with a part that is not ``graph_safe`` (it reads device values on the host in its
        forward) runs eagerly whatever ``graphs`` says, and so does a model whose capture failed once."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if graphs and self.decoder.graph_safe:
            runner = self.decode_graphs(cache)
            if runner.takes(entries):
                # graphs="lazy" (the generation loop's choice): graphs of a few widths that serve every batch
                # size, each captured when it is needed for the fifth time
                return runner.run(entries, capture_after=4 if graphs == "lazy" else 0)
            return self.step_graphs(cache).run(entries)
        return run_step(self.decoder, cache, entries)

    def decode_graphs(self, cache):
        """The captured decode steps that belong to ``cache``."""
        runner = getattr(cache, "_decode_graphs", None)
        if runner is None or runner.model is not self.decoder:
            runner = DecodeGraphs(self.decoder, cache)
            cache._decode_graphs = runner
        return runner

    def step_graphs(self, cache):
        """The captured steps of other shapes that belong to ``cache``."""
        runner = getattr(cache, "_step_graphs", None)
        if runner is None or runner.model is not self.decoder:
            runner = StepGraphs(self.decoder, cache)
            cache._step_graphs = runner
        return runner

    def generator(self, cache=None, max_tokens=None, max_batch=None, use_graphs=True, ahead=True):
        """A TextGenerator over this model.  Without a cache one is made for ``max_tokens``.
        ``ahead``: with graphs, a decode step is started before the tokens of the step before it
        have reached the host (they are taken from the device), so the device does not wait for the
        host between steps."""
        if cache is None:
            cache = self.new_cache(max_tokens or min(self.spec.max_positions * 8, 1 << 16))
        return TextGenerator(lambda entries: self.step(cache, entries, graphs="lazy" if use_graphs else False), sample_rows, cache,
                             max_positions=self.spec.max_positions, vocab_size=self.spec.vocab_size,
                             default_stop_ids=self.spec.stop_token_ids, bos_token_id=self.spec.bos_token_id,
                             max_batch=max_batch, fetch=_IdFetcher(self.runtime.device), clock=_EventClock(),
                             ahead_fn=(lambda sequences, ids, rows: self._step_ahead(cache, sequences, ids, rows))
                             if use_graphs and ahead and self.decoder.graph_safe else None,
                             take_rows=lambda logits, keep: logits[torch.tensor(keep, device=logits.device)])

    def _step_ahead(self, cache, sequences, ids, rows):
        """The decode step of ``sequences`` with the tokens ``ids[rows]`` that are still on the device,
        through the graph of their width if there is one (None otherwise: a width without a graph
        runs eagerly, which needs the tokens on the host)."""
        if len(rows) != ids.numel():
            ids = ids[torch.tensor(rows, device=ids.device)]
        entries = [StepEntry(s, [0]) for s in sequences]
        return self.decode_graphs(cache).run(entries, capture_after=4, device_ids=ids)

    def generate(self, prompts, options=None, on_token=None, **option_fields):
        """Generate for one prompt (a list of ints) or many.  Options as an InferenceOptions (or
        a list of them), or as keyword fields of one."""
        if options is None:
            options = InferenceOptions(**option_fields)
        elif option_fields:
            raise ValueError("give either an InferenceOptions or keyword fields, not both")
        if self._generator is None:
            self._generator = self.generator()
        return self._generator.generate(prompts, options, on_token)


class ModelLoader:
    """The reference's loading entry point by name (src/DotLLM.Models/ModelLoader.cs:21-28)."""

    @staticmethod
    def load(folder, dtype="bfloat16", device="cuda"):
        return Model.load(folder, dtype, device)
