"""Level choice per chunk (src/utils.py:294-314 of the reference): highest level that fits, else level 0."""
from cachegen_b200.serde.adaptation import config_selection


def test_highest_level_that_fits_is_taken():
    sizes = [{1: 10_000_000, 2: 20_000_000, 3: 40_000_000}] * 4
    # 4 chunks, 1 s in all: 0.25 s per chunk.  At 1 Gbit/s the levels take 0.08 / 0.16 / 0.32 s.
    ttft, cfg = config_selection([1.0, 1.0, 2.0, 0.1], chunk_delay=0.5, slo=1.0, sizes=sizes)
    assert cfg == [2, 2, 3, 0]                     # 2 Gbit/s fits level 3 (0.16 s); 0.1 Gbit/s fits nothing
    assert abs(ttft - (0.16 + 0.16 + 0.16 + 0.5)) < 1e-12


def test_a_transfer_that_takes_exactly_its_share_does_not_fit():
    ttft, cfg = config_selection([8.0], chunk_delay=3.0, slo=1.0, sizes=[{1: 10 ** 9}])   # exactly 1 s
    assert cfg == [0] and ttft == 3.0
