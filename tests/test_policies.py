"""Choices the engine makes from sizes alone (no GPU needed)."""

from inf_engine_b200.parts.attention import decode_splits


def test_decode_splits_cover_the_keys_and_respect_the_launch_limit():
    for keys_cap in (1, 63, 64, 300, 2048, 4096, 8192, 131072, 1 << 20):
        for n_streams in (1, 8, 64, 512, 4096):
            for max_splits in (192, 384):
                n, sk = decode_splits(keys_cap, n_streams, max_splits)
                assert n * sk >= keys_cap and (n - 1) * sk < keys_cap
                assert n <= max_splits
                assert sk >= 64 and sk & (sk - 1) == 0 and sk % 32 == 0


def test_decode_splits_grow_with_the_number_of_streams():
    few = decode_splits(4096, 8)[1]
    some = decode_splits(4096, 64)[1]
    many = decode_splits(4096, 512)[1]
    assert few <= some <= many
    assert few == 64 and many == 512


def test_checking_device_errors_needs_no_device_when_nothing_was_loaded():
    import inf_engine_b200.kernels as kernels
    if kernels._stream_lib is None and kernels._tc_lib is None and kernels._fa5_lib is None:
        kernels.check_device_errors()          # nothing loaded: nothing to read, no CUDA call
