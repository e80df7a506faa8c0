"""Run (or print) a launch recipe:  python run.py <recipe> [--num-gpus N] [--mode …] [--dry-run] [-- extra train flags]."""
import argparse
import shlex
import sys

from miles_b200 import recipes
from miles_b200.utils.launch import ExecuteTrainConfig, build_command, execute_train


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    extra: list[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, extra = argv[:i], argv[i + 1:]
    p = argparse.ArgumentParser(prog="run.py")
    p.add_argument("recipe", help="a recipe name, or `list`")
    p.add_argument("--num-gpus", type=int, default=8)
    p.add_argument("--mode", choices=["normal", "debug_minimal", "debug_one_sample"], default="normal")
    p.add_argument("--hf-checkpoint", default=None)
    p.add_argument("--data", default=None)
    p.add_argument("--eval-data", default=None)
    p.add_argument("--save", default=None)
    p.add_argument("--mxfp8", action="store_true")
    p.add_argument("--true-on-policy", action="store_true")
    p.add_argument("--dynamic-sampling", action="store_true")
    p.add_argument("--use-kl-loss", action="store_true")
    p.add_argument("--wandb-project", default=None)
    p.add_argument("--master-port", type=int, default=29511)
    p.add_argument("--log-file", default=None)
    p.add_argument("--launcher", choices=["torchrun", "workers"], default="torchrun",
                   help="workers: the ranks run as a pool of the worker manager (one supervised process per rank, per-rank logs)")
    p.add_argument("--worker-log-dir", default=None)
    p.add_argument("--dry-run", action="store_true", help="print the command instead of running it")
    a = p.parse_args(argv)
    if a.recipe == "list":
        for name, fn in sorted(recipes.RECIPES.items()):
            print(f"{name:22s} {(fn.__doc__ or '').strip().splitlines()[0] if fn.__doc__ else ''}")
        return 0
    knobs = recipes.Knobs(num_gpus=a.num_gpus, mode=a.mode, hf_checkpoint=a.hf_checkpoint, data=a.data, eval_data=a.eval_data, save=a.save,
                          mxfp8=a.mxfp8, true_on_policy=a.true_on_policy, dynamic_sampling=a.dynamic_sampling, use_kl_loss=a.use_kl_loss,
                          wandb_project=a.wandb_project, extra=extra)
    r = recipes.build(a.recipe, knobs)
    cfg = ExecuteTrainConfig(num_gpus=r.num_gpus, entry=r.entry, master_port=a.master_port, env=r.env, log_file=a.log_file, dry_run=a.dry_run,
                             launcher=a.launcher, log_dir=a.worker_log_dir)
    if a.dry_run:
        print(shlex.join(build_command(r.args, cfg)))
        return 0
    return int(execute_train(r.args, cfg))


if __name__ == "__main__":
    sys.exit(main())
