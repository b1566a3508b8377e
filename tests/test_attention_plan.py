"""How a step's tokens are handed to the attention kernels, and how the decode kernel's keys are cut (host logic)."""
import random

from iitj_llm_coopt_b200.kernels import AttentionPlan


def plan_for(contexts):
    return AttentionPlan([1] * len(contexts), contexts, "cpu", items=False, tiles=False, total_tokens=len(contexts))


def test_items_and_tiles_of_a_mixed_step():
    plan = AttentionPlan([1, 200, 1, 64], [10, 700, 33, 64], "cpu", items=False, tiles=False)
    assert plan.item_rows == [0, 201] and plan.decode_pos == [9, 32]
    assert sorted(plan.tile_rows) == [(1, 64, 500, 1), (65, 64, 564, 1), (129, 64, 628, 1), (193, 8, 692, 1), (202, 64, 0, 3)]
    assert sorted(plan.big_rows) == [(1, 128, 500, 1), (129, 72, 628, 1), (202, 64, 0, 3)]
    # a step of single tokens only is recognised without walking the requests
    fast = plan_for([10, 33, 700])
    assert fast.item_rows == [0, 1, 2] and fast.decode_pos == [9, 32, 699] and fast.n_tiles == 0


def test_split_covers_every_context_up_to_the_bound():
    rng = random.Random(0)
    for _ in range(300):
        n = rng.choice([1, 2, 5, 8, 33, 64, 200])
        contexts = [rng.choice([1, 17, 64, 65, 300, 2048, 5000, 16384, 40000]) for _ in range(n)]
        for bound in (None, (max(contexts) + 512) // 512 * 512):
            for head_dim in (64, 128):
                for window in (0, 1000):
                    kps, most = plan_for(contexts).split(rng.choice([1, 2, 8]), window, 148, head_dim, bound)
                    assert kps % 64 == 0 and kps >= 64 and 1 <= most <= 64
                    top = (bound if bound is not None else max(contexts))
                    for ctx in contexts + ([top] if bound is not None else []):
                        pos = ctx - 1
                        lo = max(0, pos - window + 1) if window else 0
                        assert (pos - lo // 64 * 64) // kps + 1 <= most       # the kernel's count of splits for this token


def test_a_long_context_among_short_ones_is_cut_finely():
    kps, most = plan_for([300] * 32 + [16384]).split(8, 0, 148, 128, None)
    assert most >= 8 and kps <= 2048            # not one CTA per key/value head for 16k keys
    # contexts of equal length fill the GPU once and are cut no finer
    kps, most = plan_for([8192] * 8).split(8, 0, 148, 128, 8704)
    assert (kps, most) == (2176, 4)
    assert plan_for([8192] * 32).split(8, 0, 148, 128, 8704) == (8704, 1)     # 256 CTAs: one wave as it is
