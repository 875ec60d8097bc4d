"""The choice of kernel and tile for prompt-sized products (pure arithmetic, no GPU): what the kernels accept, and the
rules that measurements gave."""
import itertools

from kindi_b200.kernels import fast

TC_WIDTHS = {64, 128, 144, 160, 176, 192, 208, 224, 240, 256}
PAIR_WIDTHS = {64, 128, 192, 256}


def test_every_choice_is_one_the_kernels_take():
    for m, n, k, sw in itertools.product((33, 100, 256, 511, 512, 700, 2048, 5000, 9314), (48, 96, 520, 2560, 3584, 20992, 51200),
                                         (64, 200, 2560, 10496, 25600), (False, True)):
        if sw and n % 32:
            continue
        kind, bn, variant = fast._prefill_tile(m, n, k, sw)
        if kind == "tc":
            assert bn in TC_WIDTHS and variant in (1, 2)
            assert variant == 1 or m >= 256
            assert not sw or bn % 32 == 0 or n <= 64
        else:
            assert kind == "pair" and bn in PAIR_WIDTHS and variant in (True, False)
            assert m >= 512                                   # a pair's tile has 256 rows
            if variant:
                # K blocks dealt out: never with SwiGLU in the epilogue, only when a stretch is at least a tile long
                # and while both operands fit the L2
                assert not sw
                assert -(-m // 256) * -(-n // bn) >= fast.N_SM // 2
                assert (m + n) * k * 2 <= 100e6


def test_choices_at_the_benchmark_sizes():
    # 3B-shaped layer, a 2048-token prompt: what was measured fastest
    assert fast._prefill_tile(2048, 20992, 2560, True) == ("pair", 256, False)      # gate/up
    assert fast._prefill_tile(2048, 2560, 10496) == ("pair", 256, True)             # down
    assert fast._prefill_tile(2048, 3584, 2560)[0] == "tc"                          # QKV
    assert fast._prefill_tile(2048, 2560, 2560)[0] == "tc"                          # O
    # the larger layers' down products do not fit the L2: not dealt out
    for f in (13824, 25600):
        kind, _, variant = fast._prefill_tile(2048, 5120, f)
        assert not (kind == "pair" and variant)


def test_split_k_plans_of_products_with_a_few_hundred_rows():
    for m, n, k in itertools.product((129, 200, 256, 384, 511, 512, 700, 1023), (96, 520, 2560, 5120), (64, 520, 2560, 10496, 25600)):
        plan = fast._prefill_split(m, n, k)
        if plan is None:
            continue
        bn, sp = plan
        assert bn in (128, 192, 256) and 2 <= sp <= 8
        assert -(-(-(-k // 64)) // sp) >= 8                  # a split keeps at least 8 K blocks
        assert -(-m // 128) * -(-n // bn) * sp <= 2 * fast.N_SM
    assert fast._prefill_split(256, 2560, 10496) is not None and fast._prefill_split(2048, 2560, 10496) is None


def test_decode_position_splits():
    ctx = lambda b: type("Ctx", (), {"B": b})()
    assert fast.decode_splits(ctx(1), 4) == 64 and fast.decode_splits(ctx(8), 4) == 9
    assert fast.decode_splits(ctx(32), 4) == 1 and fast.decode_splits(ctx(64), 4) == 1
    assert fast.decode_splits(ctx(16), 4) == 4 and fast.decode_splits(ctx(1), 1) == 64


def test_which_gate_up_form_takes_a_small_step():
    """the decode form up to 16 rows and while the activations are a tensor of less than 128 KB, the prompt form after"""
    import torch
    form = lambda m, width, stride=None: fast._swiglu_in_decode_form(      # noqa: E731
        torch.empty((m, stride or width), dtype=torch.bfloat16)[:, :width])
    assert [form(m, 2560) for m in (1, 16, 17, 25, 26, 32, 33, 128, 129)] == [True, True, True, True, False, False, False,
                                                                              False, False]
    assert form(63, 1024) and not form(64, 1024)               # a narrower model: 2 KB a row
    assert not form(17, 5120) and form(12, 5120)               # a wider one
    assert not form(17, 2560, stride=16384)                    # rows that lie far apart: the extent counts, not the bytes read
    assert not form(200, 64)                                   # never beyond 128 rows
