"""Reward hub: `async_rm(args, sample)` dispatches on `rm_type`.

Types follow the reference (miles/rollout/rm_hub/__init__.py:31-108): `math`, `dapo`, `deepscaler`,
`gemma_math`, `f1`, `gpqa`, `ifbench`, `remote_rm`, `random`, `deterministic_random`, with a `boxed_`
prefix that first extracts the last \\boxed{…} answer; `--custom-rm-path` overrides.  Added here for
benchmarks on random-init models: `even_fraction` and `last_mod7` (rule-based synthetic rewards).
"""
from __future__ import annotations

import asyncio
import hashlib
import random
import re
import string
from collections import Counter

from ..types import Sample
from ..utils.misc import load_function


# ---- answer extraction -------------------------------------------------------------------------

def last_boxed(text: str) -> str | None:
    i = text.rfind("\\boxed")
    if i < 0:
        return None
    j = text.find("{", i)
    if j < 0:
        return None
    depth, k = 0, j
    while k < len(text):
        if text[k] == "{":
            depth += 1
        elif text[k] == "}":
            depth -= 1
            if depth == 0:
                return text[j + 1:k]
        k += 1
    return None


def normalize_math(s: str) -> str:
    s = s.strip().strip("$").replace("\\!", "").replace("\\,", "").replace("\\ ", "").replace(" ", "")
    s = s.replace("\\left", "").replace("\\right", "").replace("dfrac", "frac").replace("tfrac", "frac")
    s = re.sub(r"\\text\{(.*?)\}", r"\1", s)
    s = re.sub(r"\\mbox\{(.*?)\}", r"\1", s)
    s = s.rstrip(".").replace("\\%", "").replace("%", "")
    if s.endswith("^\\circ") or s.endswith("^{\\circ}"):
        s = s[: s.rfind("^")]
    m = re.fullmatch(r"(-?)\\frac\{(-?\d+)\}\{(-?\d+)\}", s) or re.fullmatch(r"(-?)(\d+)/(\d+)", s)
    if m and int(m.group(3)) != 0:
        num, den = int(m.group(2)) * (-1 if m.group(1) else 1), int(m.group(3))
        s = str(num // den) if num % den == 0 else repr(num / den)
    try:
        f = float(s.replace(",", ""))
        if f == int(f):
            return str(int(f))
        return repr(f)
    except ValueError:
        return s


def math_equal(pred: str | None, label: str | None) -> bool:
    if pred is None or label is None:
        return False
    return normalize_math(pred) == normalize_math(label)


def grade_math(response: str, label: str) -> float:
    ans = last_boxed(response)
    if ans is None:
        m = re.findall(r"(?:answer is|Answer:)\s*([^\n]+)", response)
        ans = m[-1] if m else None
    return 1.0 if math_equal(ans, label) else 0.0


def grade_dapo(response: str, label: str) -> dict:
    tail = response[-300:]
    m = re.findall(r"(?i)Answer\s*:\s*([^\n]+)", tail)
    pred = m[-1].strip() if m else None
    ok = math_equal(pred, label)
    return {"score": 1.0 if ok else -1.0, "acc": ok, "pred": pred}


def grade_deepscaler(response: str, label: str) -> float:
    if "</think>" in response:
        response = response.split("</think>")[-1]
    elif "<think>" in response:
        return 0.0
    return 1.0 if math_equal(last_boxed(response), label) else 0.0


def _norm_text(s: str) -> list[str]:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return s.split()


def grade_f1(response: str, label: str) -> float:
    p, g = _norm_text(response), _norm_text(label)
    if not p or not g:
        return float(p == g)
    common = Counter(p) & Counter(g)
    n = sum(common.values())
    if n == 0:
        return 0.0
    prec, rec = n / len(p), n / len(g)
    return 2 * prec * rec / (prec + rec)


def grade_gpqa(response: str, label: str) -> float:
    m = re.findall(r"(?i)answer\s*(?:is)?\s*:?\s*\(?([A-D])\)?", response)
    if not m:
        m = re.findall(r"\b([A-D])\b", response[-50:])
    return 1.0 if m and m[-1].upper() == str(label).strip().upper() else 0.0


def grade_ifbench(response: str, sample: Sample) -> float:
    """Instruction-following checks listed in sample.metadata['instructions'] (a small built-in set)."""
    checks = (sample.metadata or {}).get("instructions", [])
    if not checks:
        return 0.0
    ok = 0
    for c in checks:
        kind, arg = (c.get("type"), c.get("arg")) if isinstance(c, dict) else (c, None)
        if kind == "max_words":
            ok += len(response.split()) <= int(arg)
        elif kind == "min_words":
            ok += len(response.split()) >= int(arg)
        elif kind == "contains":
            ok += str(arg).lower() in response.lower()
        elif kind == "not_contains":
            ok += str(arg).lower() not in response.lower()
        elif kind == "lowercase":
            ok += response == response.lower()
        elif kind == "uppercase":
            ok += response == response.upper()
        elif kind == "ends_with":
            ok += response.rstrip().endswith(str(arg))
        elif kind == "json":
            import json
            try:
                json.loads(response)
                ok += 1
            except Exception:
                pass
    return ok / len(checks)


# ---- synthetic rule rewards (benchmarks on random-init weights) -----------------------------------

def even_fraction(sample: Sample) -> float:
    ids = sample.tokens[len(sample.tokens) - sample.response_length:]
    return sum(1 for t in ids if t % 2 == 0) / max(1, len(ids))


def last_mod7(sample: Sample) -> float:
    return 1.0 if sample.response_length > 0 and sample.tokens[-1] % 7 == 0 else 0.0


async def remote_rm(args, sample: Sample) -> float:
    import aiohttp

    payload = {"prompt": sample.prompt, "response": sample.response, "label": sample.label}
    async with aiohttp.ClientSession() as sess:
        async with sess.post(args.rm_url, json=payload) as resp:
            resp.raise_for_status()
            out = await resp.json()
    return out["reward"] if isinstance(out, dict) and "reward" in out else out


async def async_rm(args, sample: Sample, **kwargs):
    spec = sample.reward_spec
    custom = (spec.custom_rm_path if spec and spec.custom_rm_path else getattr(args, "custom_rm_path", None))
    if custom:
        fn = load_function(custom)
        res = fn(args, sample, **kwargs)
        return await res if asyncio.iscoroutine(res) else res
    rm_type = (spec.rm_type if spec and spec.rm_type else None) or (sample.metadata or {}).get("rm_type") or args.rm_type
    if rm_type is None:
        raise ValueError("no --rm-type / --custom-rm-path given")
    response, label = sample.response, sample.label
    if rm_type.startswith("boxed_"):
        response = last_boxed(response) or ""
        rm_type = rm_type[len("boxed_"):]
    if rm_type == "remote_rm":
        return await remote_rm(args, sample)
    if rm_type in ("math", "gemma_math"):
        return grade_math(sample.response, label) if "\\boxed" in sample.response or rm_type == "math" else float(math_equal(response, label))
    if rm_type == "dapo":
        return grade_dapo(response, label)
    if rm_type == "deepscaler":
        return grade_deepscaler(sample.response, label)
    if rm_type == "f1":
        return grade_f1(response, label or "")
    if rm_type == "gpqa":
        return grade_gpqa(response, label)
    if rm_type == "ifbench":
        return grade_ifbench(response, sample)
    if rm_type == "random":
        return float(random.randint(0, 1))
    if rm_type == "deterministic_random":
        h = hashlib.sha256(f"{sample.prompt}|{sample.response}|{sample.tokens[-8:]}".encode()).digest()
        return float(h[0] & 1)
    if rm_type == "even_fraction":
        return even_fraction(sample)
    if rm_type == "last_mod7":
        return last_mod7(sample)
    raise NotImplementedError(f"rm_type {rm_type}")


async def batched_async_rm(args, samples: list[Sample], **kwargs) -> list:
    custom = getattr(args, "custom_rm_path", None)
    if custom and getattr(args, "group_rm", False):
        fn = load_function(custom)
        res = fn(args, samples, **kwargs)
        return await res if asyncio.iscoroutine(res) else res
    return await asyncio.gather(*[async_rm(args, s, **kwargs) for s in samples])
