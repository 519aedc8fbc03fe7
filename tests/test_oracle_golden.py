"""Pin the CPU oracle to the reference's own golden vectors (no GPU).

Sources in the reference: tests/depth_one_parity.rs:31-77 (bit-exact golden test), recipe
tests/support/depth_one_reference.rs:5-61, fixtures tests/fixtures/depth_one_main*.{pssa,bin}.
"""
import struct

import numpy as np

import oracle as O


def parse_v7(data: bytes):
    """Independent pure-Python V7 reader (checkpoint.rs:1-27, 912-956) used to cross-check the oracle's loader."""
    assert data[:4] == b"PSSA"
    version, plen, csum = struct.unpack_from("<HQQ", data, 4)
    payload = data[22:]
    assert version == 7 and plen == len(payload)
    off = 0

    def u64():
        nonlocal off
        (v,) = struct.unpack_from("<Q", payload, off)
        off += 8
        return v

    def f32():
        nonlocal off
        (v,) = struct.unpack_from("<f", payload, off)
        off += 4
        return v

    def floats():
        nonlocal off
        n = u64()
        a = np.frombuffer(payload, np.float32, n, off).copy()
        off += 4 * n
        return a

    def u64s():
        nonlocal off
        n = u64()
        a = np.frombuffer(payload, np.uint64, n, off).copy()
        off += 8 * n
        return a

    def param():
        data_ = floats()
        floats(), floats(), floats()
        return data_

    out = {"checksum": csum, "payload": payload}
    out["dims"] = [u64() for _ in range(6)]
    out["hyper"] = [f32() for _ in range(7)]
    out["step"] = u64()
    out["rng"] = u64()
    nv = u64()
    vocab = []
    for _ in range(nv):
        l = u64()
        vocab.append(payload[off:off + l].decode())
        off += l
    out["vocab"] = vocab
    for name in ["embed_w", "a_mat", "w_delta", "w_b", "w_c", "w_qx", "w_qh", "w_gate", "w_proj", "mlp_w1",
                 "mlp_w2", "unembed_w", "norm_gamma", "norm_beta"]:
        out[name] = param()
    out["h_persistent"] = floats()
    out["count"], out["write_head"] = u64(), u64()
    out["keys"], out["values"], out["norm_sq"], out["confidence"] = floats(), floats(), floats(), floats()
    out["last_seen"] = u64s()
    out["ad_down"], out["ad_up"] = param(), param()
    out["ad_cons"] = floats()
    return out


NAME_TO_ID = {
    "a_mat": O.A_MAT, "w_delta": O.W_DELTA, "w_b": O.W_B, "w_c": O.W_C, "w_qx": O.W_QX, "w_qh": O.W_QH,
    "w_gate": O.W_GATE, "w_proj": O.W_PROJ, "mlp_w1": O.MLP_W1, "mlp_w2": O.MLP_W2,
    "norm_gamma": O.NORM_GAMMA, "norm_beta": O.NORM_BETA, "h_persistent": O.H_PERSISTENT,
    "keys": O.BANK_KEYS, "values": O.BANK_VALUES, "norm_sq": O.BANK_NORM_SQ, "confidence": O.BANK_CONFIDENCE,
    "ad_down": O.AD_DOWN, "ad_up": O.AD_UP, "ad_cons": O.AD_CONS,
}


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_fnv_and_loader_agree_with_independent_reader(golden_dir):
    data = (golden_dir / "depth_one_main85d9d33_initial.pssa").read_bytes()
    ref = parse_v7(data)
    assert O.lib().pssa_oracle_fnv1a64(ref["payload"], len(ref["payload"])) == ref["checksum"]
    m = O.Model.load(data)
    assert [m.d_vocab, m.d_latent, m.d_state, m.d_mem_key, m.mem_capacity, m.chunk_len] == ref["dims"]
    assert m.depth == 1 and m.tau_mem == np.float32(0.8)
    assert np.array_equal(bits(m.tensor(-1, O.EMBED)), bits(ref["embed_w"]))
    assert np.array_equal(bits(m.tensor(-1, O.UNEMBED)), bits(ref["unembed_w"]))
    for name, tid in NAME_TO_ID.items():
        assert np.array_equal(bits(m.tensor(0, tid)), bits(ref[name])), name
    assert m.bank_meta(0)[:2] == (ref["count"], ref["write_head"]) == (2, 0)
    assert np.array_equal(m.bank_last_seen(0), ref["last_seen"])


def test_rng_and_init_reproduce_the_initial_checkpoint_bit_for_bit(golden_dir):
    """SimpleRng + Xavier draw order + log-spaced A init (pssa.rs:630-690, 2019-2072) against every
    randomly initialised tensor of the reference's initial V7 fixture."""
    ref = parse_v7((golden_dir / "depth_one_main85d9d33_initial.pssa").read_bytes())
    m = O.Model.new(depth=1, d_vocab=7, d_latent=4, d_state=2, d_mem_key=2, mem_capacity=3, chunk_len=3,
                    tau_mem=0.8, seed=192)
    assert np.array_equal(bits(m.tensor(-1, O.EMBED)), bits(ref["embed_w"]))
    assert np.array_equal(bits(m.tensor(-1, O.UNEMBED)), bits(ref["unembed_w"]))
    for name in ["a_mat", "w_delta", "w_b", "w_c", "w_qx", "w_qh", "w_gate", "w_proj", "mlp_w1", "ad_down",
                 "norm_gamma", "norm_beta"]:
        assert np.array_equal(bits(m.tensor(0, NAME_TO_ID[name])), bits(ref[name])), name
    assert m.rng_state == ref["rng"]
    # the two recipe inserts (depth_one_reference.rs:34-35) reproduce keys, norm_sq and values
    m.bank_insert(0, [0.1, -0.2], [0.3, -0.2, 0.1, 0.5])
    m.bank_insert(0, [-0.2, 0.15], [-0.1, 0.4, -0.5, 0.2])
    for name in ["keys", "values", "norm_sq", "confidence"]:
        assert np.array_equal(bits(m.tensor(0, NAME_TO_ID[name])), bits(ref[name])), name


def test_chunk_forward_reproduces_golden_loss_and_logits(golden_dir):
    """Words [0,22) of the AVX2 golden: loss + 3x7 logits of forward_train_chunk([1,2,1],[2,1,3]) on the
    fresh recipe model (depth_one_reference.rs:43-48). Later words depend on backward + AdamW."""
    obs = np.frombuffer((golden_dir / "depth_one_main014f617_avx2_observed.bin").read_bytes(), np.uint32)
    assert obs.size == 67
    m = O.Model.load((golden_dir / "depth_one_main85d9d33_initial.pssa").read_bytes())
    loss, logits = m.chunk_forward([1, 2, 1], [2, 1, 3])
    got = np.concatenate([bits(np.array([loss], np.float32)), bits(logits).ravel()])
    assert np.array_equal(got, obs[:22]), (got, obs[:22])


def test_token_inference_equals_chunk_forward_rows(golden_dir):
    """tests/stacked_depth.rs:296-317: forward_inference logits equal the chunk-forward rows bitwise, so the
    golden rows above also pin forward_inference / prefill_inference."""
    data = (golden_dir / "depth_one_main85d9d33_initial.pssa").read_bytes()
    a, b, c = O.Model.load(data), O.Model.load(data), O.Model.load(data)
    _, rows = a.chunk_forward([1, 2, 1], [2, 1, 3])
    for t, tok in enumerate([1, 2, 1]):
        assert np.array_equal(bits(b.forward_inference(tok)), bits(rows[t]))
    rc, done, last = c.prefill_inference([1, 2, 1])
    assert rc == 1 and done == 3 and np.array_equal(bits(last), bits(rows[2]))
    assert np.array_equal(bits(a.state()), bits(b.state())) and np.array_equal(bits(b.state()), bits(c.state()))


def test_trained_fixture_loads(golden_dir):
    m = O.Model.load((golden_dir / "depth_one_main014f617_avx2_trained.pssa").read_bytes())
    assert m.step_counter == 2 and m.bank_meta(0)[0] >= 2
    assert np.all(np.isfinite(m.forward_inference(1)))


def test_corrupt_containers_are_rejected(golden_dir):
    import pytest
    data = bytearray((golden_dir / "depth_one_main85d9d33_initial.pssa").read_bytes())
    data[100] ^= 1
    with pytest.raises(ValueError, match="checksum"):
        O.Model.load(bytes(data))
    with pytest.raises(ValueError):
        O.Model.load(b"PSSA\x07\x00")
