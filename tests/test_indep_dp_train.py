"""`--indep-dp` in the trainer: two cells (separate torch.distributed worlds) average gradients and stay identical; when a
cell stops between steps and the membership is republished, the survivor goes on alone."""
import json
import os
import socket
import sys

import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

BASE = ("--model-name tiny --fp32 --rollout-batch-size 4 --n-samples-per-prompt 2 --rollout-max-response-len 8 "
        "--rm-type even_fraction --lr 1e-3 --colocate --advantage-estimator grpo "
        "--data-source-path miles_b200.rollout.data_source.SyntheticSource --synthetic-prompt-len 6 10")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cell(cell, n_cells, store_port, world_port, num_rollout, out_dir, leave_after):
    os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(world_port))
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=0, world_size=1)          # every cell is a world of its own
    import train as T
    from miles_b200.args import parse_args

    # a short group timeout only where a cell is meant to go missing; otherwise a loaded machine (parallel test workers)
    # must not turn a slow peer into a lost one
    extra = f" --num-rollout {num_rollout} --indep-dp-timeout {5 if leave_after is not None else 60}"
    if n_cells > 1:
        extra += f" --indep-dp --indep-dp-num-cells {n_cells} --indep-dp-cell-id {cell} --indep-dp-store 127.0.0.1:{store_port}"
    args = parse_args((BASE + extra).split())
    if leave_after is not None and cell == 1:
        args.num_rollout = leave_after                              # this cell stops between steps
    tr = T.train(args)
    w = torch.cat([p.detach().flatten().double() for p in tr.actor.model.parameters()])
    with open(os.path.join(out_dir, f"cell{cell}.json"), "w") as f:
        json.dump({"sum": float(w.sum()), "abs": float(w.abs().sum()), "rows": len(tr.history.rows),
                   "cells": getattr(tr.actor, "last_cells", None)}, f)
    if leave_after is not None and cell == 1:
        # what the controller does when a cell is gone: publish the next membership
        tr.actor.indep_dp.members.publish(1, [0])


def _run(n_cells, num_rollout, tmp, leave_after=None):
    ctx = mp.get_context("spawn")
    os.makedirs(str(tmp), exist_ok=True)
    store_port = _free_port()
    procs = [ctx.Process(target=_cell, args=(c, n_cells, store_port, _free_port(), num_rollout, str(tmp), leave_after))
             for c in range(n_cells)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    return [json.load(open(os.path.join(str(tmp), f"cell{c}.json"))) for c in range(n_cells)]


def test_two_cells_average_gradients_and_stay_identical(tmp_path):
    a, b = _run(2, 2, tmp_path)
    assert a["rows"] == b["rows"] == 2 and a["cells"] == [0, 1]
    assert abs(a["sum"] - b["sum"]) < 1e-9 and abs(a["abs"] - b["abs"]) < 1e-9       # same weights after two averaged steps
    (solo,) = _run(1, 2, tmp_path / "solo")
    assert abs(solo["abs"] - a["abs"]) > 1e-9                                         # and not the single-cell result


def test_survivor_continues_after_a_cell_leaves(tmp_path):
    a, b = _run(2, 3, tmp_path, leave_after=1)
    assert b["rows"] == 1 and a["rows"] == 3
    assert a["cells"] == [0]                                                          # the last exchange ran on the new membership
