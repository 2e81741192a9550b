"""Speculative decoding: the host logic (n-gram drafter, greedy acceptance, acceptance-rate estimate and draft window;
no GPU needed) and, on a GPU, verify rounds through exl3_step_forward's all-rows head against plain greedy decoding."""
import numpy as np
import pytest

from tests import helpers as H


def test_ngram_draft_takes_the_earliest_occurrence_of_the_longest_suffix():
    from exl3b200.spec import ngram_draft
    #      0  1  2  3  4  5  6  7  8  9 10 11
    seq = [5, 6, 7, 8, 9, 1, 6, 7, 3, 2, 6, 7]
    # suffix (6, 7) occurs at 1..3 (followed by 8 9 1) and at 6..8 (followed by 3 2): the earliest wins
    assert ngram_draft(seq, 3, 2) == [8, 9, 1]
    assert ngram_draft(seq, 10, 2) == [8, 9, 1, 6, 7, 3, 2, 6, 7]          # capped at the end of the sequence
    assert ngram_draft(seq, 3, 3) == []                                   # the longest repeated suffix has 2 tokens
    seq2 = [1, 2, 3, 4, 9, 2, 3, 4, 7, 3, 4]
    # the longest suffix that occurs earlier is (3, 4): first at 2..4, followed by 9 2
    assert ngram_draft(seq2, 2, 2) == [9, 2]
    seq3 = [4, 2, 3, 4, 2, 3, 4]
    # suffix (2, 3, 4) = positions 4..7 occurs earlier at 1..4 -> followed by 2 3 4; (4, 2, 3, 4) occurs at 0..4 too and is longer
    assert ngram_draft(seq3, 2, 2) == [2, 3]
    assert ngram_draft([1, 2, 3], 4, 2) == [] and ngram_draft([], 4, 1) == [] and ngram_draft(seq, 0, 2) == []
    assert ngram_draft([7, 7, 7, 7], 2, 1) == [7]                         # overlapping occurrences: suffix (7,7,7) at 0..3


def test_greedy_accept():
    from exl3b200.spec import greedy_accept
    assert greedy_accept([], [11]) == [11]
    assert greedy_accept([11, 12, 13], [11, 12, 13, 14]) == [11, 12, 13, 14]      # everything agreed: the bonus token too
    assert greedy_accept([11, 99, 13], [11, 12, 13, 14]) == [11, 12]             # second draft token wrong
    assert greedy_accept([99, 12, 13], [11, 12, 13, 14]) == [11]                 # first draft token wrong


def test_accept_rate_and_draft_window():
    from exl3b200.spec import AcceptRate
    r = AcceptRate(6, cost_ratio=0.1)
    assert r.draft_window() == 6                        # warm-up: full windows
    for _ in range(60):
        r.update(6, 6)                                  # everything accepted
    assert r.accept_p > 0.95 and r.draft_window() == 6
    for _ in range(200):
        r.update(0, 6)                                  # nothing accepted
    assert r.accept_p < 0.05 and r.draft_window() == 1
    r2 = AcceptRate(8, cost_ratio=0.1)
    r2.accept_p, r2.accept_obs = 0.55, 100
    w55 = r2.draft_window()
    r2.accept_p = 0.8
    assert 1 <= w55 < r2.draft_window() <= 8            # the optimum grows with the acceptance rate
    r3 = AcceptRate(1)
    assert r3.draft_window() == 1


@pytest.mark.gpu
@pytest.mark.parametrize("kv_bits", [0, 4])
def test_verify_rounds_reproduce_greedy_decoding(ctx, kv_bits):
    """Sequences decoded through verify rounds (drafts taken from the known greedy continuation with an error planted at
    a seeded position) end up with the tokens of plain one-token-per-step decoding, and every round accepts exactly the
    draft tokens before the planted error plus the model's own token.  Positions whose top-2 logits are closer than the
    fp16 noise between the two batch shapes are allowed to differ; the comparison of that sequence stops there."""
    import torch
    import exl3b200
    from exl3b200.spec import SpecSession
    from exl3b200.step import SyntheticModel
    n_layers, vocab, n_new = 2, 2048, 40
    prompts_len = [250, 33, 120]
    bsz = len(prompts_len)

    def fresh(seed=3):
        pool = exl3b200.Pool(0, n_layers, 12, 8, 128, kv_bits, kv_bits)
        model = SyntheticModel(n_layers, 1024, 16, 8, 128, 3072, vocab, K=4, cb=1, pages=12, kv_bits=kv_bits, seed=seed, pool=pool)
        return pool, model

    r = H.rng(21)
    prompts = [r.integers(0, vocab, n).astype(np.int64) for n in prompts_len]

    def prefill(pool, model):
        blocks = [pool.alloc_prefix(p, 1)[0] for p in prompts]
        pps = max(len(b) for b in blocks)
        bt = np.zeros((bsz, pps), np.int32)
        for j, b in enumerate(blocks):
            bt[j, :len(b)] = b
        sl = torch.zeros(bsz, dtype=torch.int32, device="cuda")
        tok, _ = model.step(ctx, H.to_dev(np.concatenate(prompts)), H.to_dev(np.array(prompts_len, np.int32)), sl, H.to_dev(bt),
                            max(prompts_len), advance=False)
        return blocks, tok.cpu().numpy()

    # ---- plain greedy decoding, one token per step, with the logits of every step
    pool, model = fresh()
    blocks, first = prefill(pool, model)
    sess = SpecSession(model, ctx, pool, prompts, first, blocks, num_draft_tokens=5)
    greedy_logits = [[] for _ in range(bsz)]
    for _ in range(n_new):
        acc, lg = sess.verify_round([[] for _ in range(bsz)], want_logits=True)
        for j in range(bsz):
            assert len(acc[j]) == 1
            greedy_logits[j].append(lg[j, 0].cpu().numpy())
    ctx.poll_status()
    want = [s[prompts_len[j]:] for j, s in enumerate(sess.seqs)]          # first token + n_new tokens
    assert all(len(w) == n_new + 1 for w in want)
    pool.close()

    # ---- the same through verify rounds
    pool, model = fresh()
    blocks, first2 = prefill(pool, model)
    assert np.array_equal(first, first2)
    sess = SpecSession(model, ctx, pool, prompts, first2, blocks, num_draft_tokens=5)
    alive = [True] * bsz
    rounds = 0
    while max(len(s) - prompts_len[j] for j, s in enumerate(sess.seqs)) < n_new - 6:       # every draft has 5 tokens to take
        drafts, expect = [], []
        for j, s in enumerate(sess.seqs):
            done = len(s) - prompts_len[j]                   # tokens known so far (incl. the first)
            d = [int(t) for t in want[j][done:done + 5]]
            bad = int(r.integers(0, 7))                      # 5, 6: no error planted
            if bad < len(d):
                d[bad] = (d[bad] + 1) % vocab
            drafts.append(d)
            expect.append(min(bad, len(d)) + 1)
        acc, _ = sess.verify_round(drafts)
        ctx.poll_status()
        rounds += 1
        for j in range(bsz):
            if not alive[j]:
                continue
            got = sess.seqs[j][prompts_len[j]:][:len(want[j])]
            ref = want[j][:len(got)]
            if got != ref:
                pos = next(i for i in range(len(got)) if got[i] != ref[i])
                lg = greedy_logits[j][pos - 1]
                gap = abs(lg[ref[pos]] - lg[got[pos]]) / lg.std()
                assert gap < 0.05, f"sequence {j} leaves the greedy path at token {pos} without a near-tie (gap {gap})"
                alive[j] = False
                continue
            assert len(acc[j]) == expect[j], (j, rounds, acc[j], drafts[j], expect[j])
    assert any(alive) and rounds < n_new
    assert sess.accepted_draft_tokens > 0 and sess.drafted_tokens > sess.accepted_draft_tokens
    pool.close()
