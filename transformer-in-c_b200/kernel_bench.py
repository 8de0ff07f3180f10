"""Times single kernels of libvitb200.so through its C-ABI (plain device pointers).

    python transformer-in-c_b200/kernel_bench.py attention GROUPS SEQ HEAD_DIM [--launches N]
    python transformer-in-c_b200/kernel_bench.py gemm M K N [--launches N]

attention  flash attention forward and backward: the tcgen05 kernels
           (vitb200_k_attention_tc*, head dimension 32 or 64) beside the
           streaming mma.sync kernels (vitb200_k_attention_stream*) and, for
           at most 64 tokens, the whole-group kernels (vitb200_k_attention
           without a probability matrix); head-major tensors, algorithmic
           TFLOP/s (4 S^2 hd forward, 8 S^2 hd backward per group) and GB/s
           (16 / 32 bytes per element of Q).
gemm       Y = X W forward, the gradient pair dX, dW, and the forward product
           with bias and with bias + GELU, TF32 operands on the tensor cores.

Timing: 3 untimed launches, then N (default 10) between two CUDA events on the
launching stream.  With --launches 1 nothing is timed beyond that one launch of
each kernel, which is the form to run under a profiler.  torch only owns the
device memory.
"""
import argparse
import ctypes
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SIZE = ctypes.c_size_t
TF32 = 2


def pointer(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def timed(call, launches):
    for _ in range(3 if launches > 1 else 1):
        assert call() == 0
    torch.cuda.synchronize()
    if launches <= 1:
        return float("nan")
    begin = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(launches):
        call()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / launches


def attention(lib, groups, seq, head_dim, launches):
    rows = groups * seq
    q, k, v, dout = (torch.randn(rows, head_dim, device="cuda") for _ in range(4))
    out = torch.empty(rows, head_dim, device="cuda")
    lse = torch.empty(rows, device="cuda")
    dots = torch.empty(rows, device="cuda")
    dq, dk, dv = (torch.zeros(rows, head_dim, device="cuda") for _ in range(3))
    scale = ctypes.c_float(1.0 / np.sqrt(head_dim))
    shape = (SIZE(groups), SIZE(seq), SIZE(head_dim), scale)
    head_major = (SIZE(0), SIZE(0), SIZE(1))
    calls = {}
    if seq <= 64 and head_dim in (16, 32):
        # One block per group, everything between the operand tiles and the
        # results in registers (mma.sync); probabilities are not written.
        calls["whole-group forward"] = lambda: lib.vitb200_k_attention(
            pointer(q), pointer(k), pointer(v), None, pointer(out), *shape, TF32,
            None)
        calls["whole-group backward"] = lambda: lib.vitb200_k_attention_backward(
            pointer(q), pointer(k), pointer(v), None, pointer(out), pointer(dout),
            pointer(dq), pointer(dk), pointer(dv), pointer(dots), *shape, TF32,
            None)
    tcgen05 = {
        "tcgen05 forward": lambda: lib.vitb200_k_attention_tc(
            pointer(q), pointer(k), pointer(v), pointer(out), pointer(lse), *shape,
            *head_major, None),
        "tcgen05 backward": lambda: lib.vitb200_k_attention_tc_backward(
            pointer(q), pointer(k), pointer(v), pointer(out), pointer(dout),
            pointer(lse), pointer(dq), pointer(dk), pointer(dv), pointer(dots),
            *shape, 0, SIZE(0), SIZE(0), SIZE(0), SIZE(1), None),
    }
    if head_dim in (32, 64):
        calls.update(tcgen05)
    calls.update({
        "streaming forward": lambda: lib.vitb200_k_attention_stream(
            pointer(q), pointer(k), pointer(v), pointer(out), pointer(lse), *shape,
            None),
        "streaming backward": lambda: lib.vitb200_k_attention_stream_backward(
            pointer(q), pointer(k), pointer(v), pointer(out), pointer(dout),
            pointer(lse), pointer(dq), pointer(dk), pointer(dv), pointer(dots),
            *shape, None),
    })
    forward_flops = 4.0 * groups * seq * seq * head_dim
    for name, call in calls.items():
        if launches <= 1 and name.startswith("streaming"):
            continue
        ms = timed(call, launches)
        flops = forward_flops * (2.0 if "backward" in name else 1.0)
        # Q, K, V read and O written forward; O, dO as well and three
        # gradients written backward.
        megabytes = rows * head_dim * 4 * (8 if "backward" in name else 4) / 1e6
        print(f"attention {groups} x {seq} x {head_dim} {name}: {ms:.3f} ms, "
              f"{flops / ms / 1e9:.0f} TFLOP/s, {megabytes / ms:.0f} GB/s",
              flush=True)


def gemm(lib, m, k, n, launches):
    x = torch.randn(m, k, device="cuda")
    w = torch.randn(k, n, device="cuda")
    dy = torch.randn(m, n, device="cuda")
    bias = torch.randn(n, device="cuda")
    y, y2 = torch.empty(m, n, device="cuda"), torch.empty(m, n, device="cuda")
    dx, dw = torch.zeros(m, k, device="cuda"), torch.zeros(k, n, device="cuda")
    sizes = (SIZE(m), SIZE(k), SIZE(n), TF32, None)
    calls = {
        "forward": (1.0, lambda: lib.vitb200_k_gemm(
            pointer(x), pointer(w), pointer(y), *sizes)),
        "gradient pair": (2.0, lambda: lib.vitb200_k_gemm_backward(
            pointer(x), pointer(w), pointer(dy), pointer(dx), pointer(dw), *sizes)),
        "forward + bias": (1.0, lambda: lib.vitb200_k_gemm_fused(
            pointer(x), pointer(w), pointer(y), pointer(bias), None, None, None,
            *sizes)),
        "forward + bias + GELU": (1.0, lambda: lib.vitb200_k_gemm_fused(
            pointer(x), pointer(w), pointer(y), pointer(bias), pointer(y2), None,
            None, *sizes)),
    }
    for name, (products, call) in calls.items():
        ms = timed(call, launches)
        print(f"[{m},{k}]x[{k},{n}] {name}: {ms:.3f} ms, "
              f"{products * 2.0 * m * k * n / ms / 1e9:.0f} TFLOP/s", flush=True)


def main():
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("what", choices=["attention", "gemm"])
    parser.add_argument("sizes", type=int, nargs=3)
    parser.add_argument("--launches", type=int, default=10)
    args = parser.parse_args()
    library = os.path.join(HERE, "libvitb200.so")
    if not os.path.exists(library):
        raise SystemExit(f"{library} is missing: run transformer-in-c_b200/build.py")
    lib = ctypes.CDLL(library)
    (attention if args.what == "attention" else gemm)(lib, *args.sizes, args.launches)
    print("tensor-core status", lib.vitb200_tensor_core_status())


if __name__ == "__main__":
    main()
