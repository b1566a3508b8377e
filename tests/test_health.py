"""A kernel that gave up (a bounded wait that ran out, a broken contract) leaves a code in the library's health
words, which travel to the host with the sampled ids.  The engine must stop there instead of going on sampling
from what such a kernel wrote.  Host logic only: the plain-torch kernel double reports the failure."""
import pytest

from configs import CONFIGS
from helpers import make_engine


def test_a_failed_kernel_stops_the_engine(model_dirs):
    cfg, _seed, page = CONFIGS["A"]
    eng = make_engine(model_dirs["A"], "float32", page, 32, device="cpu", max_num_seqs=4)
    seq = eng.new_sequence([5, 6, 7, 8], 6, 0.0, True)
    eng.step()
    assert len(seq.tokens) == 5                       # a healthy step hands out its token
    eng.sampler.k.health_codes = (0, (5 << 16) | 17, 0, 0)
    with pytest.raises(RuntimeError, match="gave up"):
        eng.run_until_done()
    assert len(seq.tokens) == 5                       # nothing was appended from the failed step
    # the failure was cleared when it was reported: a new engine step works again
    eng.sampler.k.health_codes = (0, 0, 0, 0)
    other = make_engine(model_dirs["A"], "float32", page, 32, device="cpu", max_num_seqs=4)
    s2 = other.new_sequence([5, 6, 7, 8], 3, 0.0, True)
    other.run_until_done()
    assert s2.finished and len(s2.tokens) == 7
