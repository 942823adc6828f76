"""Shared helpers of the GPU parity tests: run a program image through the C ABI."""
import numpy as np

from synaptik_b200 import native, program

NP_DTYPES = {program.F32: np.float32, program.I32: np.int32, program.I64: np.int64, program.BOOL: np.uint8}


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
