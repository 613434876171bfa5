"""Generates the golden fixtures: inputs and outputs of the reference's own CPU kernels (oracle/_ref,
compiled from the reference sources) for the dtypes its test-suite never exercises (fp16, bf16,
int32). Run where oracle/_ref exists:

    python tests/golden/make_golden.py

Every tensor is one `.tannic` file (the reference's own on-disk tensor record,
include/tannic/serialization.hpp:26-66, written by tannic_b200/serialization.py) named
<set>/<case>.<tensor>.tannic; complex results are stored as their [.., 2] float view, bit-packed
comparison results as their bytes (int8). Cases named *_wide hold the result
of the reference's float-accumulating instantiation on exactly up-converted operands, rounded once to
the storage type — the behaviour the device path implements; the others are the literal result.
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402
from tannic_b200 import serialization  # noqa: E402

HERE = Path(__file__).resolve().parent


def main():
    assert oracle.ref() is not None, "build oracle/_ref first (make -C oracle ref)"
    state = {"set": "reference", "count": 0, "bytes": 0}

    def put(name, **arrays):
        folder = HERE / state["set"]
        folder.mkdir(exist_ok=True)
        for k, v in arrays.items():
            path = folder / f"{name}.{k}.tannic"
            serialization.save(v, path)
            state["count"] += 1
            state["bytes"] += path.stat().st_size

    R = "ref"
    # config 2 in miniature: Z = log(X) + Y*Y - exp(X), fp16, row-broadcast Y
    x = oracle.fill((24, 64), torch.float16, 1, "uniform", 0.1, 4.0)
    y = oracle.fill((1, 64), torch.float16, 2, "uniform", -2.0, 2.0)
    z = oracle.binary("sub", oracle.binary("add", oracle.unary("log", x, impl=R), oracle.binary("mul", y, y, impl=R), impl=R),
                      oracle.unary("exp", x, impl=R), impl=R)
    put("expr_fp16", x=x, y=y, z=z)
    xb, yb = x.to(torch.bfloat16), y.to(torch.bfloat16)
    zb = oracle.binary("sub", oracle.binary("add", oracle.unary("log", xb, impl=R), oracle.binary("mul", yb, yb, impl=R), impl=R),
                       oracle.unary("exp", xb, impl=R), impl=R)
    put("expr_bf16", x=xb, y=yb, z=zb)
    # int32 column-broadcast add
    a = oracle.fill((40, 48), torch.int32, 3, "uniform", -1000, 1000)
    b = oracle.fill((40, 1), torch.int32, 4, "uniform", -1000, 1000)
    put("add_int32", a=a, b=b, z=oracle.binary("add", a, b, impl=R))
    # bf16 X . W^T: literal (bf16 accumulation) and float-accumulating instantiation
    xm = oracle.fill((3, 20, 136), torch.bfloat16, 5, "normal", 0.0, 1.0)
    w = oracle.fill((24, 136), torch.bfloat16, 6, "normal", 0.0, 0.02)
    put("gemm_bf16", x=xm, w=w, z=oracle.matmul(xm, w.t(), impl=R),
        z_wide=oracle.matmul(xm, w.t().float(), impl=R).to(torch.bfloat16))
    q = oracle.fill((2, 3, 19, 64), torch.float16, 7, "normal", 0.0, 1.0)
    k = oracle.fill((2, 3, 19, 64), torch.float16, 8, "normal", 0.0, 1.0)
    s = oracle.matmul(q, k.transpose(-1, -2).float(), impl=R).to(torch.float16)
    put("scores_fp16", q=q, k=k, s_wide=s, s_scaled=oracle.scale(s, 0.125, impl=R))
    # fp16 conv 3x3 pad 1 and 1x1, literal and float instantiation
    xc = oracle.fill((2, 16, 9, 8), torch.float16, 9, "normal", 0.0, 1.0)
    w3 = oracle.fill((8, 16, 3, 3), torch.float16, 10, "normal", 0.0, 0.1)
    w1 = oracle.fill((24, 16, 1, 1), torch.float16, 11, "normal", 0.0, 0.3)
    bias = oracle.fill((8,), torch.float16, 12, "uniform", -1.0, 1.0)
    put("conv_fp16", x=xc, w3=w3, w1=w1, bias=bias,
        y3=oracle.conv2d(xc, w3, 1, 1, impl=R), y3_wide=oracle.conv2d(xc.float(), w3.float(), 1, 1, impl=R).to(torch.float16),
        y3b_wide=oracle.conv2d(xc.float(), w3.float(), 1, 1, bias=bias.float(), impl=R).to(torch.float16),
        y1_wide=oracle.conv2d(xc.float(), w1.float(), 1, 0, impl=R).to(torch.float16),
        y3s2_wide=oracle.conv2d(xc.float(), w3.float(), 2, 1, impl=R).to(torch.float16))
    # bf16 row reductions over 197 columns
    sr = oracle.fill((6, 197), torch.bfloat16, 13, "normal", 0.0, 1.0)
    put("reduce_bf16", s=sr, argmax=oracle.reduce("argmax", sr, -1, impl=R), argmin=oracle.reduce("argmin", sr, -1, impl=R),
        sum=oracle.reduce("sum", sr, -1, impl=R), mean=oracle.reduce("mean", sr, -1, impl=R),
        sum_wide=oracle.reduce("sum", sr.float(), -1, impl=R).to(torch.bfloat16),
        argmax_axis0=oracle.reduce("argmax", sr, 0, impl=R))
    # fp16 / int32 conv1d: literal and float instantiation
    x1 = oracle.fill((2, 6, 23), torch.float16, 14, "normal", 0.0, 1.0)
    k1 = oracle.fill((5, 6, 4), torch.float16, 15, "normal", 0.0, 0.3)
    xi, ki = oracle.fill((1, 3, 11), torch.int32, 16, "uniform", -9, 9), oracle.fill((2, 3, 3), torch.int32, 17, "uniform", -3, 3)
    put("conv1d", x=x1, k=k1, y_s2p1=oracle.conv1d(x1, k1, 2, 1, impl=R), y_s2p1_wide=oracle.conv1d(x1.float(), k1.float(), 2, 1, impl=R).to(torch.float16),
        xi=xi, ki=ki, yi=oracle.conv1d(xi, ki, 1, 0, impl=R))
    # comparisons: bit-packed boolean results (bytes stored as int8)
    ca_, cb_ = oracle.fill((5, 13), torch.bfloat16, 18, "uniform", -2, 2), oracle.fill((5, 13), torch.bfloat16, 19, "uniform", -2, 2)
    cb_[0], cb_[3, 4:9] = ca_[0], ca_[3, 4:9]
    ca_[1, 2] = float("nan")
    put("compare_bf16", a=ca_, b=cb_, **{n: oracle.compare_packed(n, ca_, cb_, impl=R)[0].view(torch.int8) for n in oracle.COMPARE})
    print(f"{state['count']} tensors -> {HERE / state['set']} ({state['bytes']} bytes)")

    # ---- data movement around the path (a folder of its own) ----
    state.update(set="data_movement", count=0, bytes=0)
    xr = oracle.fill((3, 4, 5), torch.bfloat16, 20, "uniform", -4, 4)
    put("repeat_bf16", x=xr, axis1_x3=oracle.repeat(xr, 3, 1, impl=R), axis0_x2=oracle.repeat(xr, 2, 0, impl=R),
        permuted_axis1_x2=oracle.repeat(xr.transpose(0, 2), 2, 1, impl=R))
    ca, cb, cc = (oracle.fill(shape, torch.float16, seed, "uniform", -4, 4) for shape, seed in (((3, 4, 5), 21), ((3, 2, 5), 22), ((3, 4, 7), 23)))
    ma, mb = oracle.fill((6, 4), torch.int32, 24, "uniform", -100, 100), oracle.fill((5, 4), torch.int32, 25, "uniform", -100, 100)
    put("concat", a=ca, b=cb, c=cc, ab_axis1=oracle.concat(ca, cb, 1, impl=R), ac_axis2=oracle.concat(ca, cc, 2, impl=R),
        m=ma, n=mb, mn_axis0=oracle.concat(ma, mb, 0, impl=R))
    tf, ti = oracle.fill((5, 7), torch.float32, 26, "uniform", -4, 4), oracle.fill((6, 6), torch.int64, 27, "uniform", -100, 100)
    put("triangular", f=tf, i=ti, f_triu0=oracle.triangular(tf, True, 0, impl=R), f_tril1=oracle.triangular(tf, False, 1, impl=R),
        i_triu2=oracle.triangular(ti, True, 2, impl=R), i_tril0=oracle.triangular(ti, False, 0, impl=R))
    oa, ob = oracle.fill((6,), torch.float32, 28, "uniform", -2, 2), oracle.fill((9,), torch.float32, 29, "uniform", -2, 2)
    ia, ib = oracle.fill((5,), torch.int64, 30, "uniform", -100, 100), oracle.fill((4,), torch.int64, 31, "uniform", -100, 100)
    put("outer", a=oa, b=ob, ab=oracle.outer(oa, ob, impl=R), ia=ia, ib=ib, iab=oracle.outer(ia, ib, impl=R))
    rho, theta = oracle.fill((3, 1, 4), torch.float32, 32, "uniform", 0, 2), oracle.fill((1, 5, 4), torch.float32, 33, "uniform", -3, 3)
    put("complex", rho=rho, theta=theta, cartesian=torch.view_as_real(oracle.complex_pair(rho, theta, False, impl=R)),
        polar=torch.view_as_real(oracle.complex_pair(rho, theta, True, impl=R)))
    print(f"{state['count']} tensors -> {HERE / state['set']} ({state['bytes']} bytes)")


if __name__ == "__main__":
    main()
