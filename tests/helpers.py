"""Shared helpers of the GPU parity tests: run a program image through the C ABI."""
import json
import os

import numpy as np

from synaptik_b200 import native, program

NP_DTYPES = {program.F32: np.float32, program.I32: np.int32, program.I64: np.int64, program.BOOL: np.uint8,
             program.BF16: np.uint16, program.F16: np.uint16}      # 16-bit storage travels as raw bit patterns


def run_image(context, builder: program.GraphBuilder, feeds, engine: int | None = None):
    """Builds the image, uploads ``feeds`` (arrays in feed order), runs, returns the publications."""
    if engine is not None:
        context.set_option("gemm_engine", engine)
    try:
        image = builder.build()
        exe = native.Executable(context, image)
    finally:
        if engine is not None:
            context.set_option("gemm_engine", 0)
    inputs, outputs = [], []
    try:
        for index, array in zip(builder.feeds, feeds):
            value = builder.values[index]
            array = np.ascontiguousarray(array, dtype=NP_DTYPES[value.dtype])
            inputs.append(context.upload(array))
        for index in builder.publications:
            outputs.append(context.buffer(max(builder.values[index].nbytes, 4)))
        exe.run(inputs, outputs)
        results = []
        for index, buf in zip(builder.publications, outputs):
            value = builder.values[index]
            results.append(buf.download(NP_DTYPES[value.dtype], value.shape))
        return results
    finally:
        exe.close()
        for b in inputs + outputs:
            b.close()


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in binary32 units in the last place (sign-magnitude aware)."""
    ia = np.ascontiguousarray(a, dtype=np.float32).view(np.int32).astype(np.int64)
    ib = np.ascontiguousarray(b, dtype=np.float32).view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    return np.abs(ia - ib)


def report(name: str, table) -> None:
    """Writes a test's measured figures as JSON into the folder SYNAPTIK_TEST_REPORT_DIR names (when it
    is set), so that stated tolerances can be compared with what a run actually measured."""
    folder = os.environ.get("SYNAPTIK_TEST_REPORT_DIR")
    if not folder:
        return
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, f"parity_{name}.json"), "w") as out:
        json.dump(table, out, indent=1)


def trajectory_distance(got, want, start, lr: float, step: int) -> dict:
    """How far two optimizer trajectories are apart after `step` steps: the relative L2 distance of the
    cumulative updates (p - p0), the share of entries further apart than a tenth of lr * step (the
    furthest Adam can have moved them is about lr * step), mean and maximum absolute difference."""
    got, want, start = (np.asarray(a, dtype=np.float32).ravel() for a in (got, want, start))
    drift = np.abs(got - want)
    moved = float(np.linalg.norm((want - start).astype(np.float64)))
    apart = float(np.linalg.norm((got - want).astype(np.float64)))
    return {"relative_l2": apart / moved if moved > 0 else (0.0 if apart == 0 else float("inf")),
            "share_apart": float(np.mean(drift > 0.1 * lr * step)), "mean": float(drift.mean()), "max": float(drift.max())}
