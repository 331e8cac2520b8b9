"""Writes tests/golden/golden.json: the known-answer vectors that pin the hot path.

Two kinds of entry:

* ``literal`` -- input/expected arrays transcribed from the assertions of the
  reference's own Zig unit tests (each entry cites the file:line of the test
  it comes from; paths are relative to the zigrad source tree).
* ``torch``   -- the loss cases of src/nn/tests/test_loss.py:42-58 and
  tests/src/loss.zig:12-54, whose expected numbers the reference regenerates
  with torch at test time (CrossEntropyLoss / SmoothL1Loss); they are
  regenerated here the same way, never typed in.

Run: python tests/golden/make_golden.py   (needs torch; CPU is enough)
"""
import json
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bmm_cases():
    r12 = list(range(1, 13))
    r24 = list(range(1, 25))
    src = "src/ndarray.zig:1067-1202"
    return [
        dict(src=src, a=[1, 2, 0, 1], a_shape=[2, 2], b=[1, 1, 1, 1], b_shape=[2, 2],
             c=[3, 3, 1, 1], c_shape=[2, 2]),
        dict(src=src, a=[1, 2, 3, 4, 5, 6], a_shape=[2, 3], b=[1, 0, 0, 1, 0, 0], b_shape=[3, 2],
             c=[1, 2, 4, 5], c_shape=[2, 2]),
        dict(src=src, a=r12[:6], a_shape=[1, 2, 3], b=r12[:6], b_shape=[1, 3, 2],
             c=[22, 28, 49, 64], c_shape=[1, 2, 2]),
        dict(src=src, a=r12, a_shape=[2, 2, 3], b=r12, b_shape=[2, 3, 2],
             c=[22, 28, 49, 64, 220, 244, 301, 334], c_shape=[2, 2, 2]),
        dict(src=src, a=r12, a_shape=[2, 2, 3], b=r12[:6], b_shape=[3, 2],
             c=[22, 28, 49, 64, 76, 100, 103, 136], c_shape=[2, 2, 2]),
        dict(src=src, a=r12, a_shape=[2, 2, 3], b=r12[:6], b_shape=[1, 3, 2],
             c=[22, 28, 49, 64, 76, 100, 103, 136], c_shape=[2, 2, 2]),
        dict(src=src, a=r12, a_shape=[1, 2, 2, 3], b=r12[:6], b_shape=[3, 2],
             c=[22, 28, 49, 64, 76, 100, 103, 136], c_shape=[1, 2, 2, 2]),
        dict(src=src, a=r12, a_shape=[2, 1, 2, 3], b=r12[:6], b_shape=[3, 2],
             c=[22, 28, 49, 64, 76, 100, 103, 136], c_shape=[2, 1, 2, 2]),
        dict(src=src, a=r24, a_shape=[2, 2, 2, 3], b=r12, b_shape=[2, 3, 2],
             c=[22, 28, 49, 64, 220, 244, 301, 334, 130, 172, 157, 208, 544, 604, 625, 694],
             c_shape=[2, 2, 2, 2]),
    ]


def bmm_bwd_cases():
    sq = "src/ndtensor.zig:1872-1922"
    ns = "src/ndtensor.zig:1943-2011"
    t1 = list(range(1, 13))
    t1t = [1, 4, 2, 5, 3, 6, 7, 10, 8, 11, 9, 12]
    t2 = [1, 0, 0, 1, 1, 1, 0, 1, 1, 0, 1, 1]
    t2t = [1, 0, 1, 0, 1, 1, 0, 1, 1, 1, 0, 1]
    ga = [1, 1, 2] * 4
    gat = [1, 1, 1, 1, 2, 2] * 2
    gb = [5, 5, 7, 7, 9, 9, 17, 17, 19, 19, 21, 21]
    gbt = [5, 7, 9, 5, 7, 9, 17, 19, 21, 17, 19, 21]
    out = []
    for ta, tb, g2 in ((0, 0, [4, 4, 6, 6]), (1, 0, [3, 3, 7, 7]), (0, 1, [4, 6, 4, 6]), (1, 1, [3, 7, 3, 7])):
        out.append(dict(src=sq, a=[1, 2, 3, 4], a_shape=[2, 2], b=[1, 0, 0, 1], b_shape=[2, 2],
                        ta=ta, tb=tb, grad_a=[1, 1, 1, 1], grad_b=g2))
    out.append(dict(src=ns, a=t1, a_shape=[2, 2, 3], b=t2, b_shape=[2, 3, 2], ta=0, tb=0, grad_a=ga, grad_b=gb))
    out.append(dict(src=ns, a=t1t, a_shape=[2, 3, 2], b=t2, b_shape=[2, 3, 2], ta=1, tb=0, grad_a=gat, grad_b=gb))
    out.append(dict(src=ns, a=t1, a_shape=[2, 2, 3], b=t2t, b_shape=[2, 2, 3], ta=0, tb=1, grad_a=ga, grad_b=gbt))
    out.append(dict(src=ns, a=t1t, a_shape=[2, 3, 2], b=t2t, b_shape=[2, 2, 3], ta=1, tb=1, grad_a=gat, grad_b=gbt))
    return out


def literal():
    base = [0, 1, 2, 3, 4, 5, 6, 7, 8] * 2
    plus1 = [1, 2, 3, 4, 5, 6, 7, 8, 9] * 2
    return dict(
        bmm=bmm_cases(),
        bmm_acc=dict(src="src/ndarray.zig:1226-1252", a=[1, 2, 3, 4], b=[5, 6, 7, 8], c0=[1, 1, 1, 1],
                     alpha=2.0, beta=3.0, c=[41, 47, 89, 103]),
        bmm_bwd=bmm_bwd_cases(),
        matvec=dict(src="src/ndarray.zig:1254-1278", a=[1, 2, 0, 1], x=[1, 6], y=[13, 6]),
        dot=dict(src="src/ndarray.zig:1025-1046", expected_sum=6),
        sum_along=dict(src="src/ndarray.zig:1280-1302", x=[3, 2, 4, 1], shape=[2, 2], dim=0, y=[7, 3]),
        max_along=dict(src="src/ndarray.zig:1304-1364", x=list(range(1, 25)), shape=[2, 3, 4],
                       dim0=list(range(13, 25)), dim1=[9, 10, 11, 12, 21, 22, 23, 24],
                       dim2=[4, 8, 12, 16, 20, 24]),
        gather=dict(src="src/ndarray.zig:1366-1404", x=list(range(1, 10)), shape=[3, 3],
                    index=[0, 1, 1, 2, 0, 2], index_shape=[3, 2], dim=1, y=[1, 2, 5, 6, 7, 9]),
        clip_norm=dict(src="src/ndarray.zig:911-950", x=[2, 2, 1, 4], norm=5.0, max_norm=4.0, delta=1e-6,
                       y=[1.6, 1.6, 0.8, 3.2], atol=1e-5),
        clamp=dict(src="src/ndtensor.zig:1551-1578", x=[-2.0, -0.5, 0.5, 2.0], lo=-1.0, hi=1.0,
                   y=[-1.0, -0.5, 0.5, 1.0], grad=[0.0, 1.0, 1.0, 0.0]),
        add_bcast=[
            dict(src="src/ndtensor.zig:1622-1656", x=base, x_shape=[2, 3, 3], y=[1, 1, 1], y_shape=[3],
                 z=plus1, grad_y=[6, 6, 6]),
            dict(src="src/ndtensor.zig:1657-1694", x=base, x_shape=[2, 3, 3], y=[1] * 6, y_shape=[2, 1, 3],
                 z=plus1, grad_y=[3] * 6),
        ],
        div_bwd=dict(src="src/ndtensor.zig:1835-1853", a=[4, 9], b=[2, 3], grad_a=[0.5, 1.0 / 3.0],
                     grad_b=[-1.0, -1.0]),
        mul_add_bwd=dict(src="src/ndtensor.zig:1789-1833", w=[3, 2], b=[1, 1], x=[4, 4], grad_w=[4, 4],
                         grad_b=[1, 1]),
        inplace_add=dict(src="src/ndtensor.zig:2153-2208", x=[4, 4, 4, 4], seed_grad=2.0, grads=[2, 2, 2, 2]),
        # eps of the backward = the library default (src/zigrad.zig:70)
        pow=dict(src="src/ndtensor.zig:2286-2312", x=[2, 3, 0, 1], exp=2.0, eps=1e-12, y=[4, 9, 0, 1], grad=[4, 6, 0, 2]),
        sqrt=dict(src="src/ndtensor.zig:2314-2340", x=[4, 9, 16, 1], eps=1e-12, y=[2, 3, 4, 1],
                  grad=[0.25, 1.0 / 6.0, 0.125, 0.5]),
    )


def torch_cases():
    def smce(inp, tgt):
        inp = torch.tensor(inp, requires_grad=True)
        tgt = torch.tensor(tgt)
        loss = torch.nn.CrossEntropyLoss()(inp, tgt)
        loss.backward()
        return dict(shape=list(inp.shape), input=inp.detach().flatten().tolist(), target=tgt.flatten().tolist(),
                    loss=float(loss.item()), input_grad=inp.grad.flatten().tolist())

    def sl1(inp, tgt, beta):
        inp = torch.tensor(inp, requires_grad=True)
        tgt = torch.tensor(tgt)
        loss = torch.nn.SmoothL1Loss(beta=beta)(inp, tgt)
        loss.backward()
        return dict(shape=list(inp.shape), input=inp.detach().flatten().tolist(), target=tgt.flatten().tolist(),
                    beta=beta, loss=float(loss.item()), input_grad=inp.grad.flatten().tolist())

    return dict(
        src="src/nn/tests/test_loss.py:42-58; tests/src/loss.zig:12-54 (abs 1e-4 loss, rel 1e-4 grad)",
        softmax_crossentropy_1d=smce([1.0, 2.0, 3.0, 4.0], [0.0, 1.0, 0.0, 0.0]),
        softmax_crossentropy_2d=smce([[1.0, 2.0, 3.0], [4.0, 1.0, 2.0]], [[1.0, 0.0, 0.0], [0.0, 1.0, 0.0]]),
        smooth_l1=sl1([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], [[2.0, 2.0, 2.0], [4.0, 4.0, 4.0]], 1.0),
    )


if __name__ == "__main__":
    out = dict(literal=literal(), torch=torch_cases(), torch_version=torch.__version__)
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote golden.json")
