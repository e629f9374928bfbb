"""The sampling kernel against the plain restatement of FeLLM's sampler."""
import math

import pytest
import torch

import plain_lfm2 as P
from fellm_b200.sampling import GenParams, Sampler

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def probs_of(sampler, logits, params, slot=0, draw=0):
    toks, probs = sampler.sample(logits.to(DEV), [(slot, p, draw) for p in params], return_probs=True)
    return toks.cpu().tolist(), probs.cpu()


@pytest.mark.parametrize("V", [515, 5000, 65536])
def test_greedy_is_first_argmax(V):
    s = Sampler(V, 4, 8, DEV)
    logits = torch.randn(3, V)
    logits[1, 17] = logits[1, 400] = 50.0                  # a tie: the lower id wins
    logits[2, V - 1] = 60.0
    toks, _ = probs_of(s, logits, [GenParams.greedy()] * 3)
    assert toks == [int(torch.argmax(logits[0])), 17, V - 1]
    toks, _ = probs_of(s, logits, [GenParams(temperature=0.8, top_k=1, repetition_penalty=1.0)] * 3)
    assert toks[1] == 17


@pytest.mark.parametrize("V", [515, 65536])
@pytest.mark.parametrize("kw", [dict(temperature=1.0, top_k=0), dict(temperature=0.7, top_k=40),
                                dict(temperature=1.3, top_k=0, top_p=0.9), dict(temperature=1.0, top_k=80, top_p=0.5),
                                dict(temperature=0.9, top_k=0, min_p=0.05), dict(temperature=1.1, top_k=50, min_p=0.1, top_p=0.8),
                                dict(temperature=0.2, top_k=80)])
def test_processed_distribution_matches_the_plain_sampler(V, kw):
    torch.manual_seed(V)
    s = Sampler(V, 4, 8, DEV)
    logits = torch.randn(2, V) * 3
    logits[1, :10] = 9.0                                   # ten tied leaders: lower ids are kept first
    p = GenParams(repetition_penalty=1.0, **kw)
    toks, probs = probs_of(s, logits, [p, p])
    for r in range(2):
        want = P.sample_distribution(logits[r], **kw)
        assert torch.equal(probs[r] > 0, want > 0), (kw, r, int((probs[r] > 0).sum()), int((want > 0).sum()))
        assert torch.allclose(probs[r], want, rtol=1e-4, atol=1e-7)
        assert probs[r][toks[r]] > 0


def test_draws_follow_the_distribution_and_the_seed():
    V = 1000
    s = Sampler(V, 4, 64, DEV)
    logits = torch.randn(1, V) * 2
    p = GenParams(temperature=1.0, top_k=8, repetition_penalty=1.0, seed=123)
    want = P.sample_distribution(logits[0], temperature=1.0, top_k=8)
    counts = torch.zeros(V)
    n = 4000
    batch = logits.repeat(50, 1).to(DEV)
    for i in range(n // 50):
        toks = s.sample(batch, [(0, p, i * 50 + j) for j in range(50)]).cpu()
        counts.index_add_(0, toks.long(), torch.ones(50))
    assert torch.equal(counts > 0, want > 0) or (counts > 0).sum() <= (want > 0).sum()      # top-k membership
    assert float((counts / n - want).abs().max()) < 0.03
    a = s.sample(batch[:4], [(0, p, 7)] * 4).cpu().tolist()
    b = s.sample(batch[:4], [(0, p, 7)] * 4).cpu().tolist()
    c = s.sample(batch[:4], [(0, GenParams(temperature=1.0, top_k=8, repetition_penalty=1.0, seed=124), 7)] * 4).cpu().tolist()
    assert a == b and len(set(a)) == 1                      # same seed and draw index: same token
    many = [s.sample(batch[:1], [(0, p, d)]).item() for d in range(40)]
    assert len(set(many)) > 1 and c is not None             # other draw indices: other tokens


def test_penalties_and_bias():
    V = 300
    s = Sampler(V, 4, 8, DEV)
    p = GenParams(temperature=0.0, repetition_penalty=2.0, frequency_penalty=0.5, presence_penalty=0.25,
                  logit_bias={7: 1.5})
    s.start_request(2, [5, 5, 9, 11], p)                   # history: 5 twice, 9, 11
    logits = torch.zeros(1, V)
    logits[0, 5], logits[0, 9], logits[0, 11], logits[0, 7], logits[0, 20] = 4.0, -1.0, 3.0, 1.0, 1.2
    # adjusted (sampling.rs:554-586): 5 -> 4/2 - 0.5*2 - 0.25 = 0.75; 9 -> -1*2 - 0.5 - 0.25 = -2.75;
    # 11 -> 3/2 - 0.5 - 0.25 = 0.75; 7 -> 1 + 1.5 = 2.5; 20 -> 1.2
    toks, probs = probs_of(s, logits, [p], slot=2)
    assert toks == [7]
    assert int(s.counts[2, 7]) == 1 and int(s.counts[2, 5]) == 2          # the sampled token joins the history
    q = GenParams(temperature=1.0, top_k=0, repetition_penalty=2.0, frequency_penalty=0.5, presence_penalty=0.25)
    s.start_request(1, [5, 5, 9, 11], q)
    _, probs = probs_of(s, logits, [q], slot=1)
    adj = logits[0].clone()
    adj[5], adj[9], adj[11] = 0.75, -2.75, 0.75
    assert torch.allclose(probs[0], torch.softmax(adj, 0), rtol=1e-4, atol=1e-7)
    s.start_request(1, [3], GenParams.greedy())             # the slot's history starts again
    assert int(s.counts[1].sum()) == 0


@pytest.mark.parametrize("V", [515, 65536, 70001])
def test_greedy_fast_path_equals_the_general_kernel(V):
    s = Sampler(V, 4, 16, DEV)
    logits = torch.randn(9, V)
    logits[3, 100] = logits[3, V - 1] = 40.0                # tie across chunks: the lower id
    logits[4, :] = -float("inf")
    fast = s.sample(logits.to(DEV), [(0, GenParams.greedy(), 0)] * 9).cpu().tolist()
    slow, _ = s.sample(logits.to(DEV), [(0, GenParams.greedy(), 0)] * 9, return_probs=True)
    assert fast == slow.cpu().tolist()
    assert fast[3] == 100 and fast[4] == 0 and fast[0] == int(torch.argmax(logits[0]))
