"""Names shared by the three scripts of this folder."""

import argparse
import os

D_MODEL = {"70m": 512, "160m": 768, "410m": 1024, "1b": 2048, "1.4b": 2048, "2.8b": 2560, "6.9b": 4096, "12b": 5120}
DEFAULT_STEPS = "step1000,step4000,step16000,step32000,step64000,step96000,step128000,step143000"


def arguments(**extra) -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--size", default="160m", choices=sorted(D_MODEL))
    p.add_argument("--layer", type=int, default=6)
    p.add_argument("--steps", default=DEFAULT_STEPS, help="comma-separated snapshot revisions of the model repository")
    p.add_argument("--root", default=os.path.expanduser("~/crosscoder"), help="caches, results and the embedded database go below")
    for name, kw in extra.items():
        p.add_argument("--" + name.replace("_", "-"), **kw)
    args = p.parse_args()
    args.steps = args.steps.split(",")
    args.hook = f"blocks.{args.layer}.hook_resid_post"
    return args


def cache_dir(args, step: str, target: str) -> str:
    return os.path.join(args.root, f"activations-{target}", f"pythia-{args.size}", step)
