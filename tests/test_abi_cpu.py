"""Host-side checks that need no GPU: the shim loads, exports every declared symbol, validates
images and lowers the reference's node lists to the expected fused launches."""
import ctypes
import os
import re
import struct

import pytest

from synaptik_b200 import build as build_module
from synaptik_b200 import native, program

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(native.DEFAULT_LIBRARY):
        build_module.build()
    return native.library()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "synaptik_cuda.h")).read()
    declared = sorted(set(re.findall(r"SYNAPTIK_CUDA_API\s+\w+\s+(synaptik_cuda_\w+)\s*\(", header)))
    assert len(declared) >= 30
    assert sorted(native.SYMBOLS) == declared
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.synaptik_cuda_abi_version() == 1


def test_no_device_means_no_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    handle = ctypes.c_void_p()
    status = lib.synaptik_cuda_context_create(ctypes.c_int32(0), ctypes.byref(handle))
    assert status == 2 and not handle.value          # NO_DEVICE, output cell stays NULL
    assert lib.synaptik_cuda_context_release(None) == 1
    assert lib.synaptik_cuda_buffer_release(None) == 1
    assert lib.synaptik_cuda_executable_run(None, 0, None, 0, None) == 1


def test_training_graph_lowers_to_fused_launches(lib):
    g = program.mlp_training_graph([784, 4096, 4096, 4096, 10], 8192, "ce")
    plan = native.describe(g.image).strip().split("\n")
    gemms = [p for p in plan if p.startswith("gemm")]
    assert len(gemms) == 4 + 4 + 3                      # forward, dW per layer, dX for layers 2..4
    assert sum("bias relu" in p for p in gemms) == 3    # ADD and RELU ride in the GEMM epilogue
    assert sum("relu_gate" in p for p in gemms) == 3    # WHERE(GT(z,0),g,0) rides in the dX epilogue
    assert sum("transposed_result" in p for p in gemms) == 4   # dW written as [N,K] without a copy
    assert sum("tcgen05_3xtf32" in p for p in gemms) == 3 + 3 + 2
    ce = [p for p in plan if p.startswith("cross_entropy")]
    assert len(ce) == 1 and "loss gradient" in ce[0] and "ONE_HOT" in ce[0]
    assert sum(p.startswith("colsum") for p in plan) == 4
    # nothing of the decomposed loss chain is left as a separate launch
    assert not any(p.startswith(k) for p in plan for k in ("binary", "where", "one_hot", "copy", "row_reduce", "full_sum"))
    # every gradient is published by exactly one step
    published = sorted(int(i) for p in plan for i in re.findall(r"publishes=\[(\d+)\]", p))
    assert published == list(range(9))


def test_small_mlp_uses_the_exact_kernel(lib):
    g = program.mlp_training_graph([32, 128, 1], 1024, "mse")
    plan = native.describe(g.image)
    assert "tcgen05" not in plan and plan.count("exact_simt") == 5
    assert "mse" in plan


def test_shared_preactivation_is_kept(lib):
    b = program.GraphBuilder()
    x = b.feed(program.F32, (64, 32))
    w = b.feed(program.F32, (16, 32))
    bias = b.feed(program.F32, (16,))
    _, z = b.linear(x, w, bias)
    b.publish(b.relu(z))
    b.publish(z)                                        # z is observable: it must be stored too
    plan = native.describe(b.build())
    assert "keep_preactivation" in plan


def test_malformed_images_are_rejected(lib):
    g = program.mlp_inference_graph([8, 4], 2)
    image = bytearray(g.image)
    def status_of(data):
        required = ctypes.c_uint64()
        return lib.synaptik_cuda_program_describe(bytes(data), ctypes.c_uint32(len(data)), None, ctypes.c_uint64(0), ctypes.byref(required))
    assert status_of(image) == 1                        # valid image, size probe
    bad = bytearray(image); bad[0] ^= 0xFF
    assert status_of(bad) == 9                          # GRAPH_COMPILATION_FAILED: magic
    assert status_of(image[:-4]) == 9                   # truncated
    bad = bytearray(image); struct.pack_into("<I", bad, 12, len(image) + 8)
    assert status_of(bad) == 9                          # total byte count disagrees
    # unknown operation wire code -> UNSUPPORTED_OPERATION
    bad = bytearray(image)
    node_offset = 64 + 40 * struct.unpack_from("<I", image, 16)[0]
    struct.pack_into("<I", bad, node_offset, 999)
    assert status_of(bad) == 13
    # FLOAT32-only operations refuse integer operands
    b = program.GraphBuilder()
    a = b.feed(program.I32, (4, 4)); c = b.feed(program.I32, (4, 4))
    b.publish(b._node("MATMUL", [a, c], program.F32, (4, 4)))
    assert status_of(b.build()) == 13
    # MATMUL operands above rank 4 are outside capability; batch dimensions that do not broadcast are malformed
    b = program.GraphBuilder()
    a = b.feed(program.F32, (2, 2, 2, 4, 4)); c = b.feed(program.F32, (4, 4))
    b.publish(b._node("MATMUL", [a, c], program.F32, (2, 2, 2, 4, 4)))
    assert status_of(b.build()) == 8
    b = program.GraphBuilder()
    a = b.feed(program.F32, (2, 4, 4)); c = b.feed(program.F32, (3, 4, 4))
    b.publish(b._node("MATMUL", [a, c], program.F32, (2, 4, 4)))
    assert status_of(b.build()) == 9
    # a batched product lowers to one launch per slice, a collapsible one to a single launch
    b = program.GraphBuilder()
    a = b.feed(program.F32, (2, 4, 4)); c = b.feed(program.F32, (2, 4, 4)); w = b.feed(program.F32, (4, 4))
    b.publish(b.matmul(a, c)); b.publish(b.matmul(a, w))
    plan = native.describe(b.build())
    assert plan.count("gemm") == 3 and "m=8 n=4 k=4" in plan
    # use before definition
    b = program.GraphBuilder()
    a = b.feed(program.F32, (4,))
    r = b.relu(a); b.publish(r)
    b.nodes[0].inputs[0] = r.index
    assert status_of(b.build()) == 9


def _plan(builder):
    return [line.split(" nodes=")[0] for line in native.describe(builder.build()).strip().split("\n")]


def test_loss_gradient_node_lists_lower_to_single_row_passes(lib):
    # the gradient rules' node lists (LossGradientRules.java:114-228, ReductionGradientRules.java:84-90) are
    # matched structurally: index cross entropy in its three reductions, with and without an ignore index,
    # joins its forward node in one launch; the dense-target form and both softmax kinds get one launch each
    F32, I64 = program.F32, program.I64
    for reduction in ("mean", "sum", "none"):
        for ignore in (None, -100):
            b = program.GraphBuilder()
            x, labels = b.feed(F32, (64, 256)), b.feed(I64, (64,))
            seed = b.feed(F32, (64,) if reduction == "none" else ())
            b.publish(b.index_cross_entropy(x, labels, reduction, ignore_index=ignore))
            b.publish(b.index_cross_entropy_backward(x, labels, seed, reduction, ignore_index=ignore))
            assert _plan(b) == ["cross_entropy rows=64 classes=256 loss gradient"], (reduction, ignore)
        b = program.GraphBuilder()
        x, target = b.feed(F32, (64, 256)), b.feed(F32, (64, 256))
        seed = b.feed(F32, (64,) if reduction == "none" else ())
        b.publish(b.dense_cross_entropy(x, target, reduction))
        b.publish(b.dense_cross_entropy_backward(x, target, seed, reduction))
        assert _plan(b) == ["dense_cross_entropy m=64 n=256", "dense_cross_entropy_backward m=64 n=256"], reduction
    for log_kind in (False, True):
        b = program.GraphBuilder()
        x, up = b.feed(F32, (64, 256)), b.feed(F32, (64, 256))
        y = b.log_softmax(x, 1) if log_kind else b.softmax(x, 1)
        b.publish(y)
        b.publish(b.log_softmax_backward(y, up, 1) if log_kind else b.softmax_backward(y, up, 1))
        assert _plan(b) == ["softmax m=64 n=256", "softmax_backward m=64 n=256"]
    # a chain whose intermediate is observable is left as the reference's nodes
    b = program.GraphBuilder()
    x, up = b.feed(F32, (64, 256)), b.feed(F32, (64, 256))
    y = b.softmax(x, 1)
    product = b.mul(up, y)
    b.publish(product)
    b.publish(b.mul(y, b.sub(up, b.sum(product, 1, True))))
    assert "softmax_backward m=64 n=256" not in _plan(b)
    # so is a loss gradient chain whose row mask is published: it runs as the reference's nodes
    for dense in (False, True):
        b = program.GraphBuilder()
        x = b.feed(F32, (64, 256))
        second = b.feed(F32, (64, 256)) if dense else b.feed(I64, (64,))
        seed = b.feed(F32, ())
        b.publish(b.dense_cross_entropy_backward(x, second, seed, "mean") if dense else b.index_cross_entropy_backward(x, second, seed, "mean", ignore_index=3))
        mask_shape = (64, 1) if dense else (64,)
        mask = next(n for n in b.nodes if n.op == program.OPS["EQ"] and tuple(b.values[n.outputs[0]].shape) == mask_shape)
        b.publish(b.values[mask.outputs[0]])
        plan = _plan(b)
        assert len(plan) > 10 and not any(line.startswith(("cross_entropy", "dense_cross_entropy")) for line in plan)
    # an ignore index on the loss node alone: the forward launch only, labelled by the same kernel
    b = program.GraphBuilder()
    x, labels = b.feed(F32, (64, 256)), b.feed(I64, (64,))
    b.publish(b.index_cross_entropy(x, labels, "mean", ignore_index=7))
    assert _plan(b) == ["cross_entropy rows=64 classes=256 loss"]


def test_linear_over_batch_dimensions_lowers_to_fused_products(lib):
    # Linear -> ReLU -> Linear on [batch, time, features]: the forward products keep bias / ReLU epilogues,
    # dX keeps its ReLU gate, all over batch * time rows; the weight gradients are per-slice products summed
    # over the batch on the exact engine
    F32 = program.F32
    b = program.GraphBuilder()
    x, w1, b1, w2, b2, up = (b.feed(F32, s) for s in ((4, 6, 32), (16, 32), (16,), (8, 16), (8,), (4, 6, 8)))
    wt1, z1 = b.linear(x, w1, b1)
    a1 = b.relu(z1)
    wt2, z2 = b.linear(a1, w2, b2)
    b.publish(z2)
    da1, dwt2 = b.matmul_backward(a1, wt2, up)
    dz1 = b.relu_backward(z1, da1)
    dx, dwt1 = b.matmul_backward(x, wt1, dz1)
    for v in (dx, b.permute(dwt1, (1, 0)), b.permute(dwt2, (1, 0)), b.sum_to_shape(dz1, (16,))):
        b.publish(v)
    plan = _plan(b)
    assert plan[0] == "gemm engine=exact_simt m=24 n=16 k=32 bias relu" and plan[1] == "gemm engine=exact_simt m=24 n=8 k=16 bias"
    assert "gemm engine=exact_simt m=24 n=16 k=8 relu_gate" in plan
    assert plan.count("gemm engine=exact_simt m=16 n=8 k=6") == 4 and plan.count("gemm engine=exact_simt m=32 n=16 k=6") == 4
    assert "colsum m=4 n=128" in plan and "colsum m=4 n=512" in plan and "colsum m=24 n=16" in plan
    # large enough for the tensor cores, the weight gradient is one contraction over batch * time
    b = program.GraphBuilder()
    x, up = b.feed(F32, (4, 256, 512)), b.feed(F32, (4, 256, 256))
    b.publish(b.sum_to_shape(b.matmul(b.swap_last_two(x), up), (512, 256)))
    assert _plan(b) == ["gemm engine=tcgen05_3xtf32 m=512 n=256 k=1024"]


def test_new_operations_are_validated(lib):
    F32, I32, I64, BOOL = program.F32, program.I32, program.I64, program.BOOL

    def status_of(builder):
        data = builder.build()
        required = ctypes.c_uint64()
        return lib.synaptik_cuda_program_describe(bytes(data), ctypes.c_uint32(len(data)), None, ctypes.c_uint64(0), ctypes.byref(required))

    # SOFTMAX: kinds 0 and 1 only, last axis only
    b = program.GraphBuilder(); x = b.feed(F32, (4, 8))
    b.publish(b._node("SOFTMAX", [x], F32, (4, 8), [1, 2]))
    assert status_of(b) == 13
    b = program.GraphBuilder(); x = b.feed(F32, (4, 8))
    b.publish(b._node("SOFTMAX", [x], F32, (4, 8), [0, 1]))
    assert status_of(b) == 8
    b = program.GraphBuilder(); x = b.feed(F32, (4, 8))
    b.publish(b.log_softmax(x, 1))
    assert status_of(b) == 1                                    # valid: size probe
    # dense-target cross entropy: the target has the logits' shape and FLOAT32 weights
    b = program.GraphBuilder(); x = b.feed(F32, (4, 8)); t = b.feed(F32, (4, 7))
    b.publish(b._node("DENSE_CROSS_ENTROPY", [x, t], F32, (), [1, 1]))
    assert status_of(b) == 8
    b = program.GraphBuilder(); x = b.feed(F32, (4, 8)); t = b.feed(I32, (4, 8))
    b.publish(b._node("DENSE_CROSS_ENTROPY", [x, t], F32, (), [1, 1]))
    assert status_of(b) == 13
    b = program.GraphBuilder(); x = b.feed(F32, (4, 8)); t = b.feed(F32, (4, 8))
    b.publish(b._node("DENSE_CROSS_ENTROPY", [x, t], F32, (4,), [1, 1]))       # MEAN publishes one value
    assert status_of(b) == 9
    # index cross entropy: the ignore flag is 0 or 1
    b = program.GraphBuilder(); x = b.feed(F32, (4, 8)); t = b.feed(I64, (4,))
    b.publish(b._node("INDEX_CROSS_ENTROPY", [x, t], F32, (), [1, 1, 2, 0]))
    assert status_of(b) == 13
    # integer operands only for SUB and EQ, and both of one type; SCALAR_SUB not on BOOL
    b = program.GraphBuilder(); p = b.feed(I32, (4,)); q = b.feed(I32, (4,))
    b.publish(b._node("ADD", [p, q], I32, (4,)))
    assert status_of(b) == 13
    b = program.GraphBuilder(); p = b.feed(I32, (4,)); q = b.feed(I64, (4,))
    b.publish(b._node("EQ", [p, q], BOOL, (4,)))
    assert status_of(b) == 9
    b = program.GraphBuilder(); p = b.feed(I64, (4,)); q = b.feed(I64, (4,))
    b.publish(b.eq(b.sub(p, q), b.scalar_sub(p, 3)))
    assert status_of(b) == 1
    b = program.GraphBuilder(); p = b.feed(BOOL, (4,))
    b.publish(b._node("SCALAR_SUB", [p], BOOL, (4,), [1]))
    assert status_of(b) == 13
    # SUM_TO_SHAPE sums leading dimensions only
    b = program.GraphBuilder(); x = b.feed(F32, (2, 3, 4))
    b.publish(b._node("SUM_TO_SHAPE", [x], F32, (3, 1)))
    assert status_of(b) == 8
    b = program.GraphBuilder(); x = b.feed(F32, (2, 3, 4))
    b.publish(b.sum_to_shape(x, (3, 4)))
    assert status_of(b) == 1


def test_unobserved_nodes_are_not_launched(lib):
    # the reference's compiler removes nodes nothing observes before a backend sees the graph; an image
    # that still holds some (here an unused dX product and an unused elementwise chain) does not launch them
    F32 = program.F32
    b = program.GraphBuilder()
    x, w, up = b.feed(F32, (64, 32)), b.feed(F32, (16, 32)), b.feed(F32, (64, 16))
    wt = b.permute(w, (1, 0))
    _, dwt = b.matmul_backward(x, wt, up)
    b.publish(b.permute(dwt, (1, 0)))
    b.relu(b.add(x, x))
    assert _plan(b) == ["gemm engine=exact_simt m=32 n=16 k=64 transposed_result"]


@pytest.mark.parametrize("activation,name", [("tanh", "TANH"), ("sigmoid", "SIGMOID"), ("silu", "SILU"), ("gelu_tanh", "GELU_TANH_APPROXIMATION"), ("gelu", "GELU")])
def test_the_other_activations_ride_in_the_gemm_epilogue_too(lib, activation, name):
    # the CPU backend's epilogue vocabulary (CpuMatmulIr.java:96-101): bias, then one terminal activation
    g = program.mlp_inference_graph([784, 4096, 4096, 10], 8192, activation=activation)
    plan = native.describe(g.image).strip().split("\n")
    assert not any(p.startswith("unary") for p in plan), plan
    assert sum(f"bias act={name}" in p and "tcgen05_3xtf32" in p for p in plan) == 2
    # training: TANH / SIGMOID differentiate through the stored activation, SILU / GELU through the stored
    # pre-activation, which the product then writes beside the activation
    g = program.mlp_training_graph([784, 4096, 4096, 10], 8192, "ce", activation=activation)
    plan = native.describe(g.image).strip().split("\n")
    fused = [p for p in plan if f"act={name}" in p]
    assert len(fused) == 2 and not any(p.startswith("unary") and f"op={name}" in p for p in plan), plan
    keeps = sum("keep_preactivation" in p for p in fused)
    assert keeps == (0 if activation in ("tanh", "sigmoid") else 2), plan


def test_16_bit_storage_lowers_to_the_f16_tensor_core_kernel_and_is_validated(lib):
    # Model.compute on BFLOAT16 / FLOAT16 storage: every Linear is one product with bias and activation in
    # its epilogue, the wide ones and the 10-class head on the tensor cores (kind::f16), no split passes
    for dtype, tag in ((program.BF16, "bf16"), (program.F16, "f16")):
        g = program.mlp_inference_graph([784, 4096, 4096, 10], 8192, True, dtype=dtype)
        plan = native.describe(g.image).strip().split("\n")
        assert [p.split(" nodes=")[0] for p in plan[:3]] == [
            f"gemm engine=tcgen05_f16 m=8192 n=4096 k=784 {tag} bias relu", f"gemm engine=tcgen05_f16 m=8192 n=4096 k=4096 {tag} bias relu",
            f"gemm engine=tcgen05_f16 m=8192 n=10 k=4096 {tag} bias"]
        assert plan[3].startswith("arg_max")
    # a contraction that is not a multiple of 8 elements has no 16-byte row pitch for TMA: the exact kernel
    g = program.mlp_inference_graph([100, 4100, 10], 8192, dtype=program.BF16)
    plan = native.describe(g.image).strip().split("\n")
    assert "engine=exact_simt" in plan[0] and "engine=exact_simt" in plan[1]
    # outside the inference path 16-bit values are refused, not silently widened
    b = program.GraphBuilder()
    x = b.feed(program.BF16, (4, 8))
    b.publish(b.softmax(x, 1))
    status = lib.synaptik_cuda_program_describe(b.build(), len(b.build()), None, 0, None)
    assert status == 13
    b = program.GraphBuilder()
    b.publish(b.add(b.feed(program.BF16, (4, 8)), b.feed(program.F16, (4, 8))))
    assert lib.synaptik_cuda_program_describe(b.build(), len(b.build()), None, 0, None) == 9
