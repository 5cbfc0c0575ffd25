"""CPU-only checks of the split planner (`make_plan` in csrc/da_api.cu) through `da_plan_num_splits`, which takes
the SM count as an argument and touches no device.  The cases pin the decisions the measurements behind them led
to (B200: 148 SMs); a planner change that moves one of them should come with a new measurement."""
import ctypes
import os

import pytest

SMS = 148  # B200


def plan(cabi, batch, head_q, head_k, dim, dim_v, max_seq_k, total_k=0, mla=False, num_splits=0, page_size=0):
    a = cabi.DecodeArgs()
    a.struct_size = ctypes.sizeof(cabi.DecodeArgs)
    a.is_bf16 = 1
    dummy = 0x1000  # never dereferenced by the planner; 16-byte aligned and not NULL
    a.q = a.k = a.o = dummy
    a.v = None if mla else dummy
    a.cu_seq_k = dummy
    a.batch, a.head_q, a.head_k, a.dim, a.dim_v = batch, head_q, head_k, dim, dim_v
    a.max_seq_k = max_seq_k
    a.total_k = total_k
    a.num_splits = num_splits
    if page_size:
        a.block_table = dummy
        a.page_size = page_size
        a.block_table_stride = (max_seq_k + page_size - 1) // page_size
    return cabi.plan_num_splits(a, SMS)


@pytest.fixture(autouse=True)
def no_overrides(monkeypatch):
    # (the library reads its environment overrides once per process: these tests assume none is set)
    if os.environ.get("DA_NUM_SPLITS") or os.environ.get("DA_KERNEL"):
        pytest.skip("planner overrides are set in the environment")


def test_invalid_arguments_give_minus_one(native_lib):
    assert plan(native_lib, 0, 32, 8, 128, 128, 4096) == -1
    assert native_lib.plan_num_splits(native_lib.DecodeArgs(), SMS) == -1  # struct_size 0


def test_forced_split_count_is_kept(native_lib):
    assert plan(native_lib, 4, 32, 32, 128, 128, 4096, num_splits=5) == 5


def test_headline_config_runs_unsplit(native_lib):
    # BASELINE config 2: 256 ragged sequences x 8 KV heads = 2048 units on 444 CTA slots, launched longest first
    assert plan(native_lib, 256, 32, 8, 128, 128, 4096, total_k=592409) == 1
    assert plan(native_lib, 256, 32, 8, 128, 128, 4096) == 1  # (the hint is not needed for it)
    assert plan(native_lib, 256, 32, 8, 128, 128, 4096, page_size=16) == 1


def test_uniform_batches_of_a_few_waves_are_split_in_two(native_lib):
    assert plan(native_lib, 128, 32, 8, 128, 128, 4096, total_k=128 * 4096) == 2  # 1024 units, lengths equal
    # the same batch, ragged (mean length well under the maximum): unsplit
    assert plan(native_lib, 128, 32, 8, 128, 128, 4096, total_k=128 * 2300) == 1
    assert plan(native_lib, 128, 32, 8, 128, 128, 4096) == 2  # without the hint nothing is known about the lengths


def test_one_long_sequence_gets_one_wave_of_chunks(native_lib):
    assert plan(native_lib, 1, 32, 32, 128, 128, 131072) == 13  # BASELINE config 5: 32 units x 13 = 416 of 444 slots
    assert plan(native_lib, 1, 32, 32, 128, 128, 16384) == 13  # its share on one of 8 GPUs


def test_short_sequences_weigh_setup_and_merge(native_lib):
    assert plan(native_lib, 4, 32, 32, 128, 128, 1024) == 3  # BASELINE config 1
    assert plan(native_lib, 8, 32, 32, 128, 128, 1024) == 1  # 256 units: a second wave costs more than it saves
    assert plan(native_lib, 2, 32, 32, 128, 128, 2048) == 6


def test_tensor_core_shapes(native_lib):
    assert plan(native_lib, 128, 32, 1, 128, 128, 2048, total_k=128 * 2048) == 1  # BASELINE config 3 (MQA-32)
    for batch, want in ((128, 1), (32, 2), (8, 8), (1, 8)):  # BASELINE config 4 (latent KV, 128 heads)
        assert plan(native_lib, batch, 128, 1, 576, 512, 4096, total_k=batch * 4096, mla=True) == want


def test_ragged_batch_of_few_latent_kv_sequences_is_split_with_the_hint(native_lib):
    lens = [2048, 2000] + [64 + 7 * i for i in range(58)]
    assert plan(native_lib, 60, 128, 1, 576, 512, 2048, mla=True) == 1
    assert plan(native_lib, 60, 128, 1, 576, 512, 2048, total_k=sum(lens), mla=True) > 1
    # more sequences than CTA-pair slots: the launch order balances them, no extra splits
    assert plan(native_lib, 128, 128, 1, 576, 512, 8192, total_k=128 * 4300, mla=True) == 1
