"""The plain implementation against the reference's hand-worked numbers (docs/05-transformer-math.md)."""
import math

import torch

from tests.plain import qwen3_plain as P


def close(a, b, tol=2e-3):
    return torch.allclose(torch.as_tensor(a, dtype=torch.float32), torch.as_tensor(b, dtype=torch.float32), atol=tol)


def test_rmsnorm_worked_example():
    # docs/05:283-290: x = [2, -4, 4, 2], g = [1, 1, 2, 1], eps = 0 -> [0.632, -1.265, 2.530, 0.632]
    y = P.rmsnorm(torch.tensor([2., -4., 4., 2.]), torch.tensor([1., 1., 2., 1.]), 0.0)
    assert close(y, [0.632, -1.265, 2.530, 0.632])


def test_rope_relative_position():
    # docs/05:509-524: one pair with frequency 1; key at 2, query at 5: score cos 3 = -0.990, also after +10
    def rotated(p):
        cos, sin = torch.tensor([[math.cos(p)]]), torch.tensor([[math.sin(p)]])
        return P.apply_rope(torch.tensor([[[1.0, 0.0]]]), cos, sin)[0, 0]
    assert close(rotated(2), [-0.416, 0.909])
    assert abs(float(rotated(5) @ rotated(2)) - math.cos(3)) < 1e-6
    assert abs(float(rotated(15) @ rotated(12)) - math.cos(3)) < 1e-6


def test_rope_table_is_theta_power():
    cos, sin = P.rope_table([0, 1, 7], 4, 10000.0)
    assert close(cos[2], [math.cos(7.0), math.cos(7.0 / 100.0)], 1e-6)
    assert close(sin[1], [math.sin(1.0), math.sin(0.01)], 1e-6)


def test_attention_worked_example():
    # docs/05:578-588: q = [1, 1]; three keys / values -> w = [0.097, 0.097, 0.806], out = [4.13, 4.13]
    k = torch.tensor([[1., 0.], [0., 1.], [2., 2.]])[:, None, :]
    v = torch.tensor([[1., 0.], [0., 1.], [5., 5.]])[:, None, :]
    q = torch.tensor([[9., 9.], [9., 9.], [1., 1.]])[:, None, :]  # only the last row's output is checked
    out = P.causal_gqa_attention(q, k, v, 1.0 / math.sqrt(2))
    assert close(out[2], [4.13, 4.13], 5e-3)


def test_attention_window_and_groups():
    torch.manual_seed(0)
    T, H, Hkv, hd = 9, 4, 2, 8
    q, k, v = torch.randn(T, H, hd), torch.randn(T, Hkv, hd), torch.randn(T, Hkv, hd)
    full = P.causal_gqa_attention(q, k, v, 0.3).reshape(T, H, hd)
    win = P.causal_gqa_attention(q, k, v, 0.3, window=3).reshape(T, H, hd)
    assert torch.allclose(full[:3], win[:3])          # the first rows see everything either way
    # row 8 with window 3 = full attention over keys 6..8 only
    sub = P.causal_gqa_attention(q[6:9], k[6:9], v[6:9], 0.3).reshape(3, H, hd)
    assert torch.allclose(win[8], sub[2], atol=1e-6)
    # heads 0, 1 read kv head 0; heads 2, 3 read kv head 1
    k2 = k.clone()
    k2[:, 1] *= 2.0
    changed = P.causal_gqa_attention(q, k2, v, 0.3).reshape(T, H, hd)
    assert torch.allclose(changed[:, :2], full[:, :2]) and not torch.allclose(changed[:, 2:], full[:, 2:])


def test_swiglu_worked_example():
    # docs/05:749-768
    xb = torch.tensor([[1.0, 2.0]])
    gate = torch.tensor([[1.0, 0.0], [-0.5, 0.5], [-1.0, -1.0]])
    up = torch.tensor([[0.0, 1.0], [1.0, 1.0], [2.0, 1.5]])
    down = torch.tensor([[1.0, 0.0, 1.0], [0.0, 0.5, -1.0]])
    assert close(P.silu(torch.tensor([1.0, 0.5, -3.0])), [0.731, 0.311, -0.142])
    assert close(P.swiglu_feed_forward(xb, gate, up, down)[0], [0.751, 1.178])


def test_tied_head_worked_example():
    # docs/05:892-903
    E = torch.tensor([[0.2, -1.0, 0.5], [0.9, 0.1, -0.3], [0.8, 0.2, -0.2], [-0.7, 0.6, 0.9]])
    assert close(P.linear(torch.tensor([[0.8, 0.3, -0.4]]), E)[0], [-0.34, 0.87, 0.78, -0.74])


def test_argmax_takes_the_lowest_index_among_equals():
    assert P.argmax_lowest(torch.tensor([0.5, 2.0, 2.0, -1.0])) == 1


def test_sampling_weights_and_draw():
    logits = torch.tensor([1.0, 3.0, 2.0, 3.0, -5.0])
    idx, w = P.sampling_weights(logits, 1.0, top_k=3)
    assert idx.tolist() == [1, 3, 2] and close(w, [1.0, 1.0, math.exp(-1.0)], 1e-6)
    idx, w = P.sampling_weights(logits, 0.5, top_p=0.7)
    assert idx.tolist() == [1, 3]                      # 2 of equal weight reach 0.7 of the mass
    idx, w = P.sampling_weights(logits, 1.0, min_p=0.5)
    assert idx.tolist() == [0, 1, 2, 3, 4] and w.tolist()[0] == 0.0 and w.tolist()[4] == 0.0
    assert P.draw(idx, w, 0.0) == 1 and P.draw(idx, w, 0.999) == 3


def test_schedule_names_a_layer_twice():
    from tests.helpers import model_folder, plain_logits
    from tests.tiny import random_tokens
    folder = model_folder("A")
    toks = tuple(random_tokens(12, 256, 1))
    a = plain_logits(folder, toks)
    b = plain_logits(folder, toks, ((0, None), (1, None)))
    c = plain_logits(folder, toks, ((0, None), (1, None), (1, None)))
    d = plain_logits(folder, toks, ((0, None), (1, None), (1, 1)))
    assert torch.equal(a, b) and not torch.allclose(a, c) and not torch.allclose(c, d)
