"""The seeded workload generator: deterministic, shard-consistent, with the stated distributions."""
import torch

from decoding_attention_b200 import synth


def test_same_seed_same_bits_and_shards_match_whole():
    w = synth.config_gqa_varlen(batch=6)
    q, k, v, cu = w.make("cpu")
    q2, k2, v2, _ = w.make("cpu")
    assert torch.equal(k.view(torch.int16), k2.view(torch.int16)) and torch.equal(q.view(torch.int16), q2.view(torch.int16))
    qs, ks, vs, cus = w.make("cpu", seqs=[4, 1])
    assert torch.equal(ks[:w.seq_lens[4]], k[w.cu[4]:w.cu[5]]) and torch.equal(qs[1], q[1])
    assert cus.tolist() == [0, w.seq_lens[4], w.seq_lens[4] + w.seq_lens[1]]
    qr, kr, vr, cur = w.make("cpu", key_range=(64, 192))
    assert torch.equal(vr[:128], v[w.cu[0] + 64:w.cu[0] + 192])


def test_distributions_and_lengths():
    w = synth.config_mha_small()
    _, k, _, _ = w.make("cpu")
    kf = k.float()
    assert kf.min() >= -1 and kf.max() <= 1 and abs(kf.mean().item()) < 5e-3 and abs(kf.std().item() - 3 ** -0.5) < 5e-3
    g = synth.config_gqa_varlen()
    assert g.batch == 256 and min(g.seq_lens) >= 512 and max(g.seq_lens) <= 4096
    assert g.kv_bytes() == g.total_k * 8 * 256 * 2
    m = synth.config_mla(batch=2, seq_k=64)
    q, k, v, _ = m.make("cpu")
    assert v is None and k.shape == (128, 1, 576) and abs(k.float().std().item() - 0.3) < 0.01
    assert m.kv_bytes() == 128 * 1152
