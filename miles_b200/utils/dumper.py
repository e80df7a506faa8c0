"""Tensor dumper: intermediate activations, parameters and gradients of the trainer and of the rollout engine written
to disk per phase / step / rank, and a comparison of two dump trees.

Chasing a train-vs-inference mismatch needs the same tensors from both sides.  The reference drives SGLang's dumper
from three phase switches — `--dumper-inference`, `--dumper-fwd-only`, `--dumper-fwd-bwd`, each a list of `key=value`
overrides on top of `--dumper-enable` / `--dumper-dir` — hooks the model non-intrusively, steps once per forward, dumps
weights and gradients after backward, and cleans the directory at start (miles/utils/dumper_utils.py:28-365).

Here the dumper is in-tree:

    layout   <dir>/<phase>/step{N:05d}/rank{R:03d}/{seq:05d}___{name}.pt      {"value", "meta"}
    names    layers.<i>.out, layers.<i>.attn.out, layers.<i>.mlp.out, embed.out, final_norm.out (forward hooks; layer indices
             are model-wide under pipeline parallelism), param.<name>, grad.<name> (`dump_model`)
    config   enable=0|1, filter=<regex on names>, max_numel=<int> (larger tensors keep a strided sample + exact statistics),
             steps=<first N steps only>, dump_grads=0|1

    python -m miles_b200.utils.dumper compare <dir A>/<phase> <dir B>/<phase> [--rtol 1e-2]

Engines replay CUDA graphs, which cannot run Python hooks: with the inference phase enabled the engine runs eagerly.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shutil
import sys
from dataclasses import dataclass

import torch

PHASES = ("inference", "fwd_only", "fwd_bwd")


@dataclass
class DumperConfig:
    enable: bool = False
    dir: str = "dumper"
    filter: str | None = None
    max_numel: int = 1 << 22
    steps: int | None = None
    dump_grads: bool = True

    @staticmethod
    def kv_to_dict(pairs) -> dict:
        out = {}
        for p in pairs or []:
            k, _, v = p.partition("=")
            k = k.strip().replace("-", "_")
            v = v.strip()
            if v.lower() in ("true", "false", "0", "1") and k in ("enable", "dump_grads"):
                out[k] = v.lower() in ("true", "1")
            elif k in ("max_numel", "steps"):
                out[k] = int(v)
            else:
                out[k] = v
        return out

    @staticmethod
    def for_phase(args, phase: str) -> "DumperConfig":
        """`--dumper-enable` + `--dumper-dir` overridden by the phase's own `key=value` list; a phase whose list is absent
        is off (the reference's rule: a phase is enabled by giving it a list, possibly empty)."""
        raw = getattr(args, f"dumper_{phase}", None)
        cfg = DumperConfig(enable=bool(getattr(args, "dumper_enable", False)) and raw is not None,
                           dir=os.path.join(getattr(args, "dumper_dir", "dumper") or "dumper", phase))
        for k, v in DumperConfig.kv_to_dict(raw).items():
            setattr(cfg, k, v)
        return cfg


class Dumper:
    def __init__(self, cfg: DumperConfig | None = None, rank: int | None = None):
        self.cfg = cfg or DumperConfig()
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.step_id = 0
        self.seq = 0
        self._hooks: list = []
        self._re = re.compile(self.cfg.filter) if self.cfg.filter else None
        self.written = 0

    # ---- control ---------------------------------------------------------------------------------------------
    @property
    def active(self) -> bool:
        return self.cfg.enable and (self.cfg.steps is None or self.step_id < self.cfg.steps)

    def step(self):
        self.step_id += 1
        self.seq = 0

    def cleanup(self):
        """Remove this rank's earlier dumps (every rank owns its own sub-directories, so no barrier is needed)."""
        root = self.cfg.dir
        if os.path.isdir(root):
            for s in os.listdir(root):
                d = os.path.join(root, s, f"rank{self.rank:03d}")
                if os.path.isdir(d):
                    shutil.rmtree(d, ignore_errors=True)

    # ---- writing ---------------------------------------------------------------------------------------------
    def dump(self, name: str, value, **meta):
        if not self.active or (self._re is not None and not self._re.search(name)):
            return
        if not torch.is_tensor(value):
            return
        t = value.detach()
        full_shape, n = tuple(t.shape), t.numel()
        f = t.float()
        stats = {"mean": float(f.mean()) if n else 0.0, "abs_max": float(f.abs().max()) if n else 0.0,
                 "norm": float(f.norm()) if n else 0.0}
        sampled = n > self.cfg.max_numel
        if sampled:
            stride = (n + self.cfg.max_numel - 1) // self.cfg.max_numel
            t = t.reshape(-1)[::stride]
        d = os.path.join(self.cfg.dir, f"step{self.step_id:05d}", f"rank{self.rank:03d}")
        os.makedirs(d, exist_ok=True)
        safe = name.replace("/", "_")
        torch.save({"value": t.cpu(), "meta": {"name": name, "shape": full_shape, "dtype": str(value.dtype), "sampled": sampled,
                                               "step": self.step_id, "rank": self.rank, **stats, **meta}},
                   os.path.join(d, f"{self.seq:05d}___{safe}.pt"))
        self.seq += 1
        self.written += 1

    def dump_model(self, model, with_grads: bool | None = None):
        """Parameters (and gradients: `.main_grad` where the optimizer keeps fp32 accumulators, else `.grad`)."""
        with_grads = self.cfg.dump_grads if with_grads is None else with_grads
        named = model.named_parameters_global() if hasattr(model, "named_parameters_global") else model.named_parameters()
        for n, p in named:
            self.dump(f"param.{n}", p.data)
            if with_grads:
                g = getattr(p, "main_grad", None)
                g = g if g is not None else p.grad
                if g is not None:
                    self.dump(f"grad.{n}", g)

    # ---- non-intrusive hooks ---------------------------------------------------------------------------------
    def register(self, model):
        """Forward hooks on the embedding, every decoder layer (and its attention / MLP), and the final norm."""
        lo = getattr(model, "layer_range", (0, 0))[0]

        def out_of(x):
            while isinstance(x, (tuple, list)) and x:
                x = x[0]
            return x

        def hook(name):
            return lambda mod, inp, out: self.dump(name, out_of(out))

        for i, layer in enumerate(getattr(model, "layers", [])):
            g = i + lo
            self._hooks.append(layer.register_forward_hook(hook(f"layers.{g}.out")))
            for sub in ("attn", "mlp"):
                m = getattr(layer, sub, None)
                if isinstance(m, torch.nn.Module):
                    self._hooks.append(m.register_forward_hook(hook(f"layers.{g}.{sub}.out")))
        return self

    def remove(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []


class DumperSwitch:
    """One set of hooks, three phases.  Trainer and engine may run the SAME module (colocated): whoever is about to run a
    forward selects its phase (`with switch.phase("inference"): …`), the hooks write to that phase's dumper."""

    def __init__(self, dumpers: dict[str, Dumper]):
        self.dumpers = dumpers
        self.current: Dumper | None = None
        self._hooked: set[int] = set()

    @staticmethod
    def from_args(args, rank: int | None = None) -> "DumperSwitch | None":
        if not getattr(args, "dumper_enable", False):
            return None
        ds = {ph: Dumper(DumperConfig.for_phase(args, ph), rank) for ph in PHASES}
        ds = {ph: d for ph, d in ds.items() if d.cfg.enable}
        for d in ds.values():
            d.cleanup()
        return DumperSwitch(ds) if ds else None

    def enabled(self, phase: str) -> bool:
        return phase in self.dumpers

    def dump(self, name, value, **meta):
        if self.current is not None:
            self.current.dump(name, value, **meta)

    def register(self, model):
        if id(model) in self._hooked:
            return
        self._hooked.add(id(model))
        proxy = Dumper(DumperConfig(enable=True))
        proxy.dump = self.dump                      # the hooks of `Dumper.register` route through the switch
        proxy.register(model)
        self._proxy = proxy

    def phase(self, name: str):
        switch = self

        class _Ctx:
            def __enter__(self):
                self.prev = switch.current
                switch.current = switch.dumpers.get(name)
                return switch.current

            def __exit__(self, *exc):
                switch.current = self.prev

        return _Ctx()

    def step(self):
        if self.current is not None:
            self.current.step()


# ---- comparison -------------------------------------------------------------------------------------------------------

def _index(root: str) -> dict:
    out = {}
    for step in sorted(os.listdir(root)):
        for rank in sorted(os.listdir(os.path.join(root, step))):
            d = os.path.join(root, step, rank)
            seen: dict[str, int] = {}
            for f in sorted(os.listdir(d)):
                name = f.split("___", 1)[1][:-3]
                k = seen.get(name, 0)
                seen[name] = k + 1
                out[(step, rank, name, k)] = os.path.join(d, f)
    return out


def compare(a: str, b: str, rtol: float = 1e-2) -> list[dict]:
    """Tensors present in both trees (same step, rank, name, occurrence) compared by relative L2 distance."""
    ia, ib = _index(a), _index(b)
    rows = []
    for key in sorted(set(ia) & set(ib)):
        x, y = torch.load(ia[key], weights_only=False), torch.load(ib[key], weights_only=False)
        vx, vy = x["value"].float(), y["value"].float()
        row = {"step": key[0], "rank": key[1], "name": key[2], "occurrence": key[3], "shape": list(x["meta"]["shape"])}
        if vx.shape != vy.shape:
            row.update(status="shape", rel=None, shape_b=list(y["meta"]["shape"]))
        else:
            den = float(vy.norm()) or 1.0
            rel = float((vx - vy).norm()) / den
            row.update(status="ok" if rel <= rtol else "diff", rel=rel, abs_max=float((vx - vy).abs().max()) if vx.numel() else 0.0)
        rows.append(row)
    for key in sorted(set(ia) ^ set(ib)):
        rows.append({"step": key[0], "rank": key[1], "name": key[2], "occurrence": key[3], "status": "only_a" if key in ia else "only_b"})
    return rows


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="miles_b200 dumper")
    sub = p.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("compare")
    c.add_argument("a")
    c.add_argument("b")
    c.add_argument("--rtol", type=float, default=1e-2)
    c.add_argument("--json", action="store_true")
    a = p.parse_args(argv)
    rows = compare(a.a, a.b, a.rtol)
    if a.json:
        print(json.dumps(rows))
    else:
        for r in rows:
            rel = f"{r['rel']:.3e}" if r.get("rel") is not None else "-"
            print(f"{r['status']:7s} {r['step']} {r['rank']} {r['name']}#{r['occurrence']} rel={rel}")
    bad = [r for r in rows if r["status"] != "ok"]
    print(f"{len(rows) - len(bad)} match, {len(bad)} differ or are missing", file=sys.stderr)
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
