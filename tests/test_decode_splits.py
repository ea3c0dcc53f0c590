"""How many CTAs share a row's keys in decode attention (``parts/attention.py::decode_splits``): the rule's decisions
at the shapes that the measurements behind it used (148 SMs)."""
from llm_infer_rust_b200.parts.attention import decode_splits


def test_a_grid_that_fills_the_sms_stays_whole():
    # 32 and 64 rows x 8 KV heads: whole, although two or four splits would fill the last wave better
    # (measured: 90.8 against 103.8 us, 177.5 against 182.3 us at 4,096 keys a row)
    for ctas in (130, 256, 512, 4096):
        for keys in (512, 4096, 65536):
            assert decode_splits(ctas, keys, 148) == 1


def test_small_grids_are_split_to_fill_the_sms():
    assert decode_splits(64, 4096, 148) == 2          # 8 rows x 8 KV heads: 128 CTAs, a cluster of two combines them
    assert decode_splits(32, 4096, 148) == 4
    assert decode_splits(8, 4096, 148) == 8           # one row: eight clusters of eight
    assert decode_splits(16, 4096, 148) == 7          # two rows: eight would be sixteen clusters of eight, which do not find room
    # every CTA keeps at least 512 keys
    assert decode_splits(8, 512, 148) == 1 and decode_splits(8, 1024, 148) == 2
    assert decode_splits(0, 4096, 148) == decode_splits(1, 4096, 148)
