"""Which decode-attention kernel a step takes and into how many runs it cuts a sequence
(`kernels.attention.decode_plan`): decided on the host from the batch size, the cache geometry and what
the device says it can hold, so it is tested here with a device that is made up."""
import pytest


@pytest.fixture
def plan(monkeypatch):
    from rust_inference_b200.kernels import attention, attention_tc
    monkeypatch.setattr(attention, "_sm_count", lambda: 148)
    monkeypatch.setattr(attention, "_DECODE", "auto")
    monkeypatch.delenv("RI_B200_DECODE_SPLITS", raising=False)
    held = {}

    def capacity(head_dim, n_splits):
        return held["fn"](head_dim, n_splits)
    monkeypatch.setattr(attention_tc, "decode_cluster_capacity", capacity)

    def run(n_seqs, n_kv_heads, max_seq_len, head_dim=None, fits=lambda hd, s: 10 ** 6):
        held["fn"] = fits
        return attention.decode_plan(n_seqs, n_kv_heads, max_seq_len, 64, head_dim)
    return run


def test_small_batches_take_clusters_and_large_ones_whole_sequences(plan, monkeypatch):
    assert plan(1, 4, 8192) == ("cluster", 8)            # 4 pairs: eight runs each, the most a cluster holds
    assert plan(8, 4, 8192) == ("cluster", 8)            # 32 pairs x 8 = 256 CTAs <= two per SM
    assert plan(16, 4, 8192) == ("cluster", 4)
    assert plan(32, 4, 8192) == ("cluster", 2)
    assert plan(37, 4, 8192) == ("cluster", 2)           # 148 pairs x 2 = 296
    assert plan(38, 4, 8192) == ("tma", 1)
    assert plan(64, 4, 8192) == ("tma", 1)
    assert plan(1, 4, 64) == ("tma", 1)                  # one page per sequence: nothing to cut
    assert plan(1, 4, 200) == ("cluster", 4)             # never more runs than pages


def test_runs_are_made_fewer_until_the_step_is_resident_together(plan):
    # what a B200 answers for head size 128: clusters of 2..8 CTAs it holds at once
    b200 = {2: 148, 3: 93, 4: 71, 5: 56, 6: 45, 7: 37, 8: 33}
    fits = lambda hd, s: b200[s]
    assert plan(8, 4, 8192, 128, fits) == ("cluster", 8)         # 32 clusters of eight fit (33)
    assert plan(9, 4, 8192, 128, fits) == ("cluster", 7)         # 36 clusters: seven CTAs each (37)
    assert plan(16, 4, 8192, 128, fits) == ("cluster", 4)
    # a device that holds fewer: the runs shrink; with no room for clusters at all the runs are merged
    # through scratch by a second kernel
    assert plan(8, 4, 8192, 128, lambda hd, s: 40 if s <= 4 else 8) == ("cluster", 4)
    assert plan(8, 4, 8192, 128, lambda hd, s: 8) == ("tma", 9)
    # without a head size nobody is asked
    assert plan(8, 4, 8192, None, lambda hd, s: 0) == ("cluster", 8)


def test_the_kernel_can_be_forced(plan, monkeypatch):
    from rust_inference_b200.kernels import attention
    monkeypatch.setattr(attention, "_DECODE", "cp_async")
    assert plan(8, 4, 8192) == ("cp_async", 9)
    assert plan(64, 4, 8192) == ("cp_async", 1)
    monkeypatch.setattr(attention, "_DECODE", "tma")
    assert plan(8, 4, 8192) == ("tma", 9)
