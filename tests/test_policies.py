"""Choices the engine makes from sizes alone (no GPU needed)."""

from inf_engine_b200.parts.attention import decode_splits


def test_decode_splits_cover_the_keys_and_respect_the_launch_limit():
    for keys in (1, 63, 64, 300, 2048, 2304, 4096, 8192, 131072, 1 << 20):
        for n_streams in (1, 8, 64, 512, 4096):
            for warps in (3, 6):
                n, sk = decode_splits(keys, n_streams, warps, 64)
                assert n * sk >= keys and (n - 1) * sk < keys
                assert -(-n // warps) <= 64
                assert sk >= 64 and sk % 32 == 0


def test_decode_splits_grow_with_the_number_of_streams():
    few = decode_splits(4096, 8)[1]
    some = decode_splits(4096, 64)[1]
    many = decode_splits(4096, 512)[1]
    assert few < some < many
    assert few <= 96 and many > 256


def test_decode_splits_fill_the_warps_of_a_block():
    # many streams: one block a stream, every warp with keys
    n, sk = decode_splits(2304, 512, 6)
    assert n == 6 and sk == 384
    # the measured best at batch 8: four blocks of six warps (256 of the 296 places for a block), 96 keys a warp
    assert decode_splits(2304, 64, 6) == (24, 96)
    # never more blocks than places: a second round of blocks costs more than longer splits
    for n_streams in (1, 8, 24, 64, 100, 512):
        n, sk = decode_splits(2304, n_streams, 6)
        assert -(-n // 6) * n_streams <= 296 or -(-n // 6) == 1


def test_checking_device_errors_needs_no_device_when_nothing_was_loaded():
    import inf_engine_b200.kernels as kernels
    if kernels._stream_lib is None and kernels._tc_lib is None and kernels._fa5_lib is None:
        kernels.check_device_errors()          # nothing loaded: nothing to read, no CUDA call


def test_small_requests_of_a_step_are_counted_once():
    from inf_engine_b200.engine.batch import StepContext
    ctx = StepContext(None, 16)
    ctx.host = {"q_lens": [1, 40, 2, 1], "ctx_before": [100, 0, 7, 3000]}
    assert ctx.keys_of_small_requests(4, 16) == (3, 3001)      # 1, 2 and 1 tokens of four heads each: at most 16 rows
    assert ctx.keys_of_small_requests(16, 16) == (2, 3001)
    ctx.host["ctx_before"][0] = 9999                            # the step's answer is kept: every layer asks again
    assert ctx.keys_of_small_requests(4, 16) == (3, 3001)
    graph_ctx = StepContext(None, 16)
    graph_ctx.host = {"q_lens": [1, 1]}                         # a captured step has no host copy of the lengths
    assert graph_ctx.keys_of_small_requests(4, 16) == (0, 0)


def test_graph_buckets_of_the_longest_context():
    from inf_engine_b200.engine.graphs import KEYS_STEP, keys_bucket
    last = 0
    for keys in sorted(list(range(1, 9000, 37)) + [8192, 8193, 16384, 16385, 40000, 131072, 1 << 20]):
        b = keys_bucket(keys)
        assert b >= keys and b >= last                       # holds the step's keys; never shrinks as they grow
        assert b - keys < max(KEYS_STEP, keys // 8)          # and is cut for at most an eighth more keys than there are
        last = b
    assert keys_bucket(2049) == 2304 and keys_bucket(8192) == 8192 and keys_bucket(8193) == 8704
    # a context that doubles crosses 16 buckets once it is long, not one per 256 keys
    assert len({keys_bucket(k) for k in range(32769, 65537)}) == 16
