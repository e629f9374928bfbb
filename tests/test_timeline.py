"""The grouping of the kernel timeline's per-CTA records into launches (no GPU needed)."""
import random

from fellm_b200.engine.timeline import group_records, kernel_name, Timeline


def rec(ident, blocks, begin, waited, end, marks=(0, 0, 0, 0)):
    return [ident | (blocks << 16), begin, waited, end, *marks]


def test_records_are_grouped_into_launches_in_time_order():
    records = []
    # embed_rows (id 1), 2 CTAs; then two launches of the same product (id 32 + 32*1, 3 CTAs) back to back
    records += [rec(1, 2, 1000, 1010, 2000), rec(1, 2, 1100, 1110, 2100)]
    records += [rec(64, 3, 3000 + 10 * i, 3500, 5000 + i, (3600, 0, 0, 0)) for i in range(3)]
    records += [rec(64, 3, 6000 + 10 * i, 6500 + i, 8000 + 100 * i) for i in range(3)]
    random.Random(1).shuffle(records)
    launches = group_records(records, detail=True)
    assert [(l.name, l.blocks) for l in launches] == [("embed_rows", 2), ("gemm_skinny[accumulate]", 3), ("gemm_skinny[accumulate]", 3)]
    a, b, c = launches
    assert a.begin_us == 0.0 and abs(a.end_us - 1.1) < 1e-9 and abs(a.waited_us - 0.01) < 1e-9
    assert abs(b.begin_us - 2.0) < 1e-9 and abs(b.end_us - 4.002) < 1e-9 and abs(b.marks_us[0] - 2.6) < 1e-9
    assert abs(c.waited_us - 5.5) < 1e-9 and abs(c.end_us - 7.2) < 1e-9 and len(c.ctas) == 3
    assert "gemm_skinny[accumulate]" in Timeline.table(launches)


def test_overlapping_launches_of_one_kernel_come_apart_by_their_cta_count():
    # a programmatic dependent starts before the launch in front of it has ended
    first = [rec(13, 4, 100 + i, 150, 900 + i) for i in range(4)]
    second = [rec(13, 4, 400 + i, 950, 1500 + i) for i in range(4)]
    launches = group_records(first + second)
    assert len(launches) == 2 and all(l.name == "attention_decode" and l.blocks == 4 for l in launches)
    assert launches[1].begin_us < launches[0].end_us


def test_names():
    assert kernel_name(7) == "gemm_umma" and kernel_name(32) == "gemm_skinny[store]" and kernel_name(32 + 64) == "gemm_skinny[swiglu]"
    assert group_records([]) == []
