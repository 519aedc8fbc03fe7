"""The product's `.pssa` reader: host-only validation (runs without a GPU) and device upload (GPU)."""
import numpy as np
import pytest

import oracle as O
from helpers import fill_synthetic, write_pssa_v8
from parity import scale_err


def test_probe_reads_the_reference_fixtures_without_a_gpu(golden_dir):
    import pssa_b200
    for name in ("depth_one_main85d9d33_initial.pssa", "depth_one_main014f617_avx2_trained.pssa"):
        data = (golden_dir / name).read_bytes()
        cfg, version = pssa_b200.PSSAModel.probe_checkpoint(data)
        ref = O.Model.load(data)
        assert version == 7 and cfg["depth"] == 1
        assert [cfg["d_vocab"], cfg["d_latent"], cfg["d_state"], cfg["d_mem_key"], cfg["mem_capacity"]] == \
            [ref.d_vocab, ref.d_latent, ref.d_state, ref.d_mem_key, ref.mem_capacity]
        assert np.float32(cfg["tau_mem"]) == np.float32(ref.tau_mem)


def test_probe_rejects_corrupt_containers_with_the_reason(golden_dir):
    import pssa_b200
    data = (golden_dir / "depth_one_main85d9d33_initial.pssa").read_bytes()
    bad = bytearray(data)
    bad[100] ^= 1
    for blob, reason in ((bytes(bad), "checksum"), (b"PSSA\x07\x00", "not a PSSA"), (b"ABCD" + data[4:], "not a PSSA"),
                         (data[:-5], "payload length"), (data[:4] + b"\x09\x00" + data[6:], "unsupported checkpoint version")):
        with pytest.raises(ValueError, match=reason):
            pssa_b200.PSSAModel.probe_checkpoint(blob)


def test_version_8_writer_round_trips_through_the_oracle_reader():
    """The test-side writer is itself checked: the oracle's reader returns the tensors it was given."""
    om = O.Model.new(3, 50, 16, 4, 4, 8, seed=2)
    fill_synthetic(om, 2, bank_fill=0.5)
    om.prefill_inference(np.arange(1, 9))  # a non-zero carry
    back = O.Model.load(write_pssa_v8(om, step_counter=5))
    assert back.depth == 3 and back.step_counter == 5
    for l in range(3):
        for tid in (O.W_DELTA, O.MLP_W2, O.AD_CONS, O.BANK_VALUES, O.A_MAT):
            assert np.array_equal(back.tensor(l, tid), om.tensor(l, tid))
        assert back.bank_meta(l)[:2] == om.bank_meta(l)[:2]
    assert np.array_equal(back.state(), om.state())


@pytest.mark.gpu
def test_fixture_loads_onto_the_device_and_reproduces_the_oracle(golden_dir):
    import pssa_b200
    gpu = pssa_b200.B200Dispatch(0)
    for name in ("depth_one_main85d9d33_initial.pssa", "depth_one_main014f617_avx2_trained.pssa"):
        data = (golden_dir / name).read_bytes()
        om = O.Model.load(data)
        gm = pssa_b200.PSSAModel.from_checkpoint(gpu, data, precision=1)
        assert np.array_equal(gm.copy_recurrent_state_to(0), om.state())  # the stored carry, bit for bit
        for tok in (1, 2, 1, 5):
            assert scale_err(gm.forward_inference(tok), om.forward_inference(tok)) <= 1e-5
        gm.close()
    gpu.close()


@pytest.mark.gpu
def test_stacked_version_8_checkpoint_with_partial_banks_and_carry():
    import pssa_b200
    gpu = pssa_b200.B200Dispatch(0)
    om = O.Model.new(3, 97, 32, 16, 8, 16, seed=4)
    fill_synthetic(om, 4, bank_fill=0.6)
    om.prefill_inference((np.arange(20) * 3 + 1) % 97)
    data = write_pssa_v8(om)
    cfg, version = pssa_b200.PSSAModel.probe_checkpoint(data)
    assert version == 8 and cfg["depth"] == 3
    gm = pssa_b200.PSSAModel.from_checkpoint(gpu, data, precision=1)
    assert np.array_equal(gm.copy_recurrent_state_to(0), om.state())
    ids = (np.arange(40) * 5 + 2) % 97
    _, logits = gm.prefill_inference(ids)
    _, _, ref = om.prefill_inference(ids)
    assert scale_err(logits, ref) <= 1e-5
    # a payload that passes the container checks but ends early inside the last array is refused before any upload
    import struct
    payload = data[22:-16]
    h = 0xcbf29ce484222325
    for byte in payload:
        h = ((h ^ byte) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    cut = b"PSSA" + struct.pack("<HQQ", 8, len(payload), h) + payload
    pssa_b200.PSSAModel.probe_checkpoint(cut)  # the header and configuration are fine
    with pytest.raises(pssa_b200.B200Error, match="invalid checkpoint: truncated while reading embed_row_marks"):
        pssa_b200.PSSAModel.from_checkpoint(gpu, cut, precision=1)
    gm.close()
    gpu.close()
