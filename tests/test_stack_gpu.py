"""The stack runner behind bench.py (rusty_b200/stack.py): what every output buffer holds after a step, against the
reference's arithmetic (dequantised f32 weights, f32 matmul), for both weight formats."""
import numpy as np
import pytest

from parity import TOL_FP32, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("native", [False, True])
@pytest.mark.parametrize("M", [1, 3])
def test_small_stack_outputs_match_the_reference_arithmetic(ctx, oracle, M, native):
    from rusty_b200 import DType
    from rusty_b200.stack import LinearStack
    from rusty_b200.workloads import StackShape
    shape = StackShape("tiny", d=256, q=256, kv=128, ffn=640, vocab=1024, layers=2)
    st = LinearStack(ctx, shape, M, DType.FP32, DType.FP32, seed=3, native=native, keep_host=True)
    assert st.native == native and not st.swiglu
    if native:
        assert set(st.plans()) == {"gemv_mma"}   # K % 128 == 0 everywhere: the re-laid-out affine format
    st.step()
    ctx.sync()
    # buffers are reused from layer to layer: each one holds the output of the LAST Linear that wrote it
    last = {}
    for i, (name, y) in enumerate(zip(st.names, st._ys)):
        last[id(y)] = i
    assert len(last) >= 4
    for i in last.values():
        x = st.host_inputs[st.dims[i][1]]
        ref = oracle.matmul_bt(x, st.host_wf[i], mt=True)
        got = np.frombuffer(st._ys[i].to_bytes(ctx), np.float32).reshape(M, st.out_n[i])
        assert rel_err(got, ref) <= TOL_FP32, st.names[i]
