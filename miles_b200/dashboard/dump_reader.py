"""Reader of the rollout dumps (`--save-debug-rollout-data`, set by `--dump-details`): per-rollout sample tables and a token
view of one sample (reference: miles/dashboard/dump_reader.py:358-895 `DumpReader`, the token and conversation views)."""
from __future__ import annotations

import glob
import os
import re

import torch


class DumpReader:
    def __init__(self, directory: str, tokenizer=None):
        self.dir, self.tokenizer = directory, tokenizer
        self._cache: dict[int, dict] = {}

    def _files(self) -> dict[int, str]:
        out = {}
        for p in glob.glob(os.path.join(self.dir, "rollout_data", "*.pt")):
            m = re.search(r"(\d+)\.pt$", p)
            if m:
                out[int(m.group(1))] = p
        return out

    def rollout_ids(self) -> list[int]:
        return sorted(self._files())

    def _load(self, rollout_id: int) -> dict:
        if rollout_id not in self._cache:
            path = self._files()[rollout_id]
            self._cache[rollout_id] = torch.load(path, weights_only=False)
            if len(self._cache) > 4:
                self._cache.pop(next(iter(self._cache)))
        return self._cache[rollout_id]

    def samples(self, rollout_id: int) -> list[dict]:
        """One row per sample: identity, lengths, reward, status, weight versions."""
        rows = []
        for gi, g in enumerate(self._load(rollout_id)["samples"]):
            for si, d in enumerate(g):
                resp = d.get("response_length") or 0
                lm = d.get("loss_mask")
                rows.append({"group": gi, "sample": si, "index": d.get("index"), "prompt_tokens": len(d.get("tokens") or []) - resp,
                             "response_tokens": resp, "trained_tokens": sum(lm) if lm else resp, "reward": d.get("reward"),
                             "status": d.get("status"), "weight_versions": d.get("weight_versions"),
                             "mean_logprob": (sum(d["rollout_log_probs"]) / max(1, len(d["rollout_log_probs"]))) if d.get("rollout_log_probs") else None})
        return rows

    def summary(self, rollout_id: int) -> dict:
        rows = self.samples(rollout_id)
        rewards = [r["reward"] for r in rows if isinstance(r["reward"], (int, float))]
        groups: dict[int, list] = {}
        for r in rows:
            if isinstance(r["reward"], (int, float)):
                groups.setdefault(r["group"], []).append(r["reward"])
        flat = sum(1 for v in groups.values() if len(v) > 1 and max(v) == min(v))
        return {"rollout_id": rollout_id, "samples": len(rows), "groups": len(groups), "groups_without_signal": flat,
                "mean_reward": sum(rewards) / len(rewards) if rewards else None,
                "mean_response_tokens": sum(r["response_tokens"] for r in rows) / max(1, len(rows)),
                "max_response_tokens": max((r["response_tokens"] for r in rows), default=0)}

    def token_view(self, rollout_id: int, group: int, sample: int) -> dict:
        d = self._load(rollout_id)["samples"][group][sample]
        toks = d.get("tokens") or []
        resp = d.get("response_length") or 0
        p = len(toks) - resp
        lm = d.get("loss_mask") or [1] * resp
        lps = d.get("rollout_log_probs") or [None] * resp
        text = [self.tokenizer.decode([t]) for t in toks] if self.tokenizer is not None else [str(t) for t in toks]
        rows = [{"pos": i, "token": t, "text": text[i], "part": "prompt"} for i, t in enumerate(toks[:p])]
        rows += [{"pos": p + j, "token": toks[p + j], "text": text[p + j], "part": "response", "trained": bool(lm[j]) if j < len(lm) else True,
                  "rollout_log_prob": lps[j] if j < len(lps) else None} for j in range(resp)]
        return {"reward": d.get("reward"), "status": d.get("status"), "tokens": rows}
