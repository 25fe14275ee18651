"""How a sum still owed to the residual stream travels from the part that left it to the norm that settles it
(parts/base.py, parts/block.py, models/causal_lm.py).  Stand-in parts on the CPU: no kernel runs here."""
from types import SimpleNamespace

from rustingstrata_b200.parts.base import Block
from rustingstrata_b200.parts.block import PreNormBlock


class Owed:
    def __init__(self):
        self.finished = 0

    def finish(self):
        self.finished += 1


class TakingNorm:
    takes_owed = True

    def __init__(self, log):
        self.log = log

    def forward(self, x, out, n_rows, rows=None, owed=None):
        self.log.append(("norm", owed))


class PlainNorm:                      # a norm that knows nothing of owed sums (no attribute, no keyword)
    def __init__(self, log):
        self.log = log

    def forward(self, x, out, n_rows, rows=None):
        self.log.append(("plain_norm", None))


class LeavingPart:
    """A mixer or feed-forward that leaves its last sum when it is allowed to."""

    def __init__(self, log, name):
        self.log, self.name = log, name

    def forward(self, h, residual, ctx, call=None):
        ctx.owed = Owed() if ctx.may_owe else None
        self.log.append((self.name, ctx.may_owe, ctx.owed))


class ObliviousPart:
    def __init__(self, log, name):
        self.log, self.name = log, name

    def forward(self, h, residual, ctx, call=None):
        self.log.append((self.name, ctx.may_owe, None))


def context():
    return SimpleNamespace(n_tokens=3, may_owe=False, owed=None, next_block_takes_owed=False)


def block(mixer_norm, mixer, ff_norm, ff):
    b = PreNormBlock.__new__(PreNormBlock)          # no runtime: only the arrangement is under test
    b.mixer_norm, b.mixer, b.ff_norm, b.feed_forward = mixer_norm, mixer, ff_norm, ff
    b.hidden = 4
    return b


class Rows(list):
    """Stands in for the scratch tensor of normed rows: any slice of it is itself."""

    def __getitem__(self, key):
        return self


def run(b, ctx):
    b.runtime = SimpleNamespace(get_scratch=lambda name: Rows())
    b.forward(object(), ctx, SimpleNamespace(mixers={"mixer": None}))


def test_a_sum_left_by_the_mixer_reaches_the_next_norm_and_nobody_else():
    log = []
    b = block(TakingNorm(log), LeavingPart(log, "mixer"), TakingNorm(log), LeavingPart(log, "ff"))
    ctx = context()
    run(b, ctx)
    (_, first), (_, allowed, left), (_, taken), (_, ff_allowed, ff_left) = log
    assert first is None                       # nothing was owed at the start
    assert allowed and left is not None and taken is left and left.finished == 0
    assert not ff_allowed and ff_left is None  # the model said nothing about the next block: the feed-forward finishes itself
    assert ctx.owed is None and ctx.may_owe is False


def test_the_last_product_of_a_block_leaves_its_sum_only_if_the_next_block_takes_it():
    log = []
    b = block(TakingNorm(log), ObliviousPart(log, "mixer"), TakingNorm(log), LeavingPart(log, "ff"))
    ctx = context()
    ctx.next_block_takes_owed = True
    run(b, ctx)
    assert log[-1][1] is True and ctx.owed is log[-1][2] and ctx.may_owe is False
    carried = ctx.owed
    log.clear()
    run(b, ctx)                                # the next block: its first norm takes what was carried over
    assert log[0] == ("norm", carried) and carried.finished == 0


def test_a_norm_that_cannot_take_the_sum_has_it_finished_first():
    log = []
    b = block(PlainNorm(log), ObliviousPart(log, "mixer"), PlainNorm(log), ObliviousPart(log, "ff"))
    assert b.first_reader_takes_owed is False
    ctx = context()
    ctx.owed = carried = Owed()                # by mistake or by a part of another kind: it must not be lost
    run(b, ctx)
    assert carried.finished == 1 and log[0] == ("plain_norm", None)
    assert [e[1] for e in log if e[0] in ("mixer", "ff")] == [False, False]      # and nobody is invited to leave one


def test_what_a_block_says_about_its_first_reader():
    log = []
    assert block(TakingNorm(log), None, PlainNorm(log), None).first_reader_takes_owed is True
    assert block(PlainNorm(log), None, TakingNorm(log), None).first_reader_takes_owed is False
    assert Block.first_reader_takes_owed.fget(SimpleNamespace()) is False       # a block of another kind: never
