"""Host logic of the SM shares two concurrent split-K weight gradients get (no GPU needed)."""
from zigrad_b200.mlp import split_sm_shares


def test_headline_step_shares():
    # 784-128 (7 output tiles) beside 128-64 (1 tile), batch 8192 = 256 k-slabs, 148 SMs:
    # 19 K ranges of 14 slabs for the first, 15 ranges of 18 slabs for the second
    assert split_sm_shares(148, 7, 1, 256) == (133, 15)


def test_shares_never_exceed_the_gpu_and_keep_whole_tiles():
    for sms in (8, 64, 132, 148):
        for t0, t1 in ((7, 1), (1, 1), (4, 2), (13, 3)):
            for slabs in (4, 32, 256, 2048):
                got = split_sm_shares(sms, t0, t1, slabs)
                if got is None:
                    assert sms < t0 + t1
                    continue
                a, b = got
                assert a % t0 == 0 and b % t1 == 0 and a >= t0 and b >= t1 and a + b <= sms
                # the second GEMM's K range is at most 1.3 times as long as the first's
                assert -(-slabs // (b // t1)) <= 1.3 * -(-slabs // (a // t0))
