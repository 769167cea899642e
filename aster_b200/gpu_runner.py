"""Execution subprocess with the command line of the reference's ``examples/_gpu_runner.py``.

The reference's examples compile in one process and execute in another
(examples/common.py:104-170): the parent saves the input and output arrays as ``.npy`` files
and passes one JSON object -- ``hsaco_path``, ``kernel_name``, ``grid``, ``block``,
``input_files``, ``output_files`` -- as the only argument; the child runs the kernel, stores
the outputs back into their files and prints ``{"times": [...]}``.  This module is that child
for the kernels of this library:

    python -m aster_b200.gpu_runner '{"kernel_name": "kernel", "input_files": [...], ...}'
"""

from __future__ import annotations

import json
import sys

import numpy as np

from .execution import InputArray, OutputArray, execute_hsaco


def run(config: dict) -> dict:
    args = [InputArray(np.load(f)) for f in config.get("input_files", [])]
    outputs = []
    for f in config.get("output_files", []):
        arr = np.load(f, allow_pickle=False)
        outputs.append(arr)
        args.append(OutputArray(arr))
    times = execute_hsaco(
        hsaco_path=config.get("hsaco_path"),
        kernel_name=config["kernel_name"],
        arguments=args,
        grid_dim=tuple(config.get("grid", (1, 1, 1))),
        block_dim=tuple(config.get("block", (64, 1, 1))),
        num_iterations=int(config.get("num_iterations", 1)),
    )
    for f, arr in zip(config.get("output_files", []), outputs):
        np.save(f, arr)
    return {"times": times}


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        print("usage: python -m aster_b200.gpu_runner '<json config>'", file=sys.stderr)
        return 2
    print(json.dumps(run(json.loads(argv[0]))))
    return 0


if __name__ == "__main__":
    sys.exit(main())
