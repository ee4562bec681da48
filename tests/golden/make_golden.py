"""Record golden vectors: run the reference's own CUDA kernels (oracle/_ref, built
by oracle/build_ref.py) on the seeded cases of cases.py and store inputs and
outputs as .npz.  Needs a GPU:

    python tests/golden/make_golden.py [output_dir]      # default: tests/golden

The committed fixtures were produced by this script on a B200."""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, ROOT)

import build_ref  # noqa: E402
import cases  # noqa: E402


def main(out_dir):
    ref = build_ref.load()
    if ref is None:
        raise SystemExit("oracle/_ref is not built: run python oracle/build_ref.py")
    dev = torch.device("cuda:0")
    os.makedirs(out_dir, exist_ok=True)
    for name, make in cases.CASES.items():
        case = make()
        outs = cases.run_reference(name, case, ref, dev)
        torch.cuda.synchronize()
        blob = {"in_" + k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in case.items()}
        blob.update({"ref_" + k: v.detach().cpu().numpy() for k, v in outs.items()})
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **blob)
        print(name, {k: tuple(v.shape) for k, v in outs.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
