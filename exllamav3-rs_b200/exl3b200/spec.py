"""Host side of speculative decoding, mirroring the reference's generator (src/generator.rs): the n-gram drafter
(get_ngram_draft, :253-270), the shared verify round (spec_verify_round, :1649-1895: all-or-nothing draft length, one
forward of q_len = drafts + 1 rows per sequence that samples every row, greedy acceptance of the longest matching prefix,
rewind by simply not advancing past the accepted tokens), the acceptance-rate estimate and the draft window derived from
it (draft_window, :1966-1993).  The device work is one exl3_step_forward with `all_rows` set."""
import numpy as np
import torch

ACCEPT_DECAY = 0.94          # src/generator.rs:1803


def ngram_draft(seq, draft_length, match_min, max_suffix=64):
    """Tokens that followed the EARLIEST earlier occurrence of the LONGEST suffix of `seq` that occurs earlier at all
    (src/generator.rs:253-270; the reference finds it with a suffix automaton, this mirror by direct search over suffixes
    of at most `max_suffix` tokens).  Empty when that suffix is shorter than match_min or draft_length <= 0."""
    n = len(seq)
    if draft_length <= 0 or match_min <= 0 or n < match_min + 1:
        return []
    a = np.asarray(seq, dtype=np.int64)
    best_end = -1
    for L in range(min(max_suffix, n - 1), match_min - 1, -1):
        suf = a[n - L:]
        # occurrences that end before the end of the sequence (an occurrence may overlap the suffix itself)
        for start in range(0, n - L):
            if a[start] == suf[0] and np.array_equal(a[start:start + L], suf):
                best_end = start + L
                break
        if best_end >= 0:
            break
    if best_end < 0:
        return []
    return [int(t) for t in a[best_end:min(best_end + draft_length, n)]]


def greedy_accept(draft, row_tokens):
    """row_tokens[i] = the model's greedy token after the fed token and the first i draft tokens.  Returns the accepted
    tokens: the model's own first token, then one more for every leading draft token it agrees with
    (src/generator.rs:1772-1781)."""
    accepted = [int(row_tokens[0])]
    for i, d in enumerate(draft):
        if int(d) != accepted[i]:
            break
        accepted.append(int(row_tokens[i + 1]))
    return accepted


class AcceptRate:
    """Running estimate of the per-token acceptance probability and the draft window that maximises expected tokens per
    unit of verify cost (src/generator.rs:1797-1806,1966-1993)."""

    def __init__(self, num_draft_tokens, cost_ratio=0.1):
        self.num_draft_tokens = int(num_draft_tokens)
        self.cost_ratio = float(cost_ratio)
        self.accept_p = 0.5
        self.accept_obs = 0

    def update(self, n_accepted_draft, window):
        a = float(n_accepted_draft)
        trials = a + (1.0 if n_accepted_draft < window else 0.0)       # one failure unless the window was exhausted
        if trials > 0.0:
            self.accept_p = self.accept_p * ACCEPT_DECAY + (a / trials) * (1.0 - ACCEPT_DECAY)
            self.accept_obs += 1

    def draft_window(self):
        nmax = self.num_draft_tokens
        if nmax <= 1 or self.accept_obs < 8:
            return nmax                                                # warm up on full windows
        r = min(max(self.cost_ratio, 0.005), 1.0)
        p = min(max(self.accept_p, 0.01), 0.999)
        best_n, best, tokens, pw = 1, -np.inf, 1.0, 1.0
        for n in range(1, nmax + 1):
            pw *= p
            tokens += pw
            score = tokens / (1.0 + n * r)
            if score > best:
                best, best_n = score, n
        return best_n


class SpecSession:
    """A batch of sequences decoded with draft verification on one model.  Each sequence keeps `seq` (all tokens, the last
    one not yet fed), its pages and kv_pos = len(seq) - 1."""

    def __init__(self, model, ctx, pool, prompts, first_tokens, blocks, num_draft_tokens=4, ngram_match_min=2):
        """`prompts`: token lists already prefilled into the pool (their KV is cached), `first_tokens`: the token sampled
        after each prompt, `blocks`: page lists the sequences hold."""
        self.model, self.ctx, self.pool = model, ctx, pool
        self.seqs = [list(map(int, p)) + [int(t)] for p, t in zip(prompts, first_tokens)]
        self.blocks = [list(b) for b in blocks]
        self.rate = AcceptRate(num_draft_tokens)
        self.ngram_match_min = ngram_match_min
        self.accepted_draft_tokens = 0
        self.drafted_tokens = 0

    def kv_pos(self, j):
        return len(self.seqs[j]) - 1

    def _ensure_pages(self, j, tokens):
        need = (tokens + 255) // 256
        while len(self.blocks[j]) < need:
            self.blocks[j] += self.pool.alloc(1)

    def ngram_drafts(self):
        w = self.rate.draft_window()
        return [ngram_draft(s, w, self.ngram_match_min) for s in self.seqs]

    def verify_round(self, drafts, want_logits=False):
        """One verify forward over all sequences.  Returns (accepted token lists, logits or None); drafts are cut to the
        shortest one (all-or-nothing, as the reference); with no draft at all this is a plain decode round."""
        bsz = len(self.seqs)
        min_len = min([self.rate.num_draft_tokens] + [len(d) for d in drafts])
        drafts = [list(d[:min_len]) for d in drafts]
        q_len = min_len + 1
        feed, seqlens = [], []
        for j in range(bsz):
            feed.append(self.seqs[j][-1])
            feed.extend(drafts[j])
            seqlens.append(self.kv_pos(j))
            self._ensure_pages(j, self.kv_pos(j) + q_len)
        pps = max(len(b) for b in self.blocks)
        bt = np.zeros((bsz, pps), np.int32)
        for j, b in enumerate(self.blocks):
            bt[j, :len(b)] = b
        dev = self.model.device
        d_ids = torch.tensor(feed, dtype=torch.int64, device=dev)
        d_q = torch.full((bsz,), q_len, dtype=torch.int32, device=dev)
        d_sl = torch.tensor(seqlens, dtype=torch.int32, device=dev)
        d_bt = torch.from_numpy(bt).to(dev)
        tok, logits = self.model.step(self.ctx, d_ids, d_q, d_sl, d_bt, q_len, advance=False, want_logits=want_logits,
                                      all_rows=True)
        rows = tok.cpu().numpy().reshape(bsz, q_len)                    # the one device-to-host copy of the round
        out = []
        for j in range(bsz):
            acc = greedy_accept(drafts[j], rows[j])
            if min_len > 0:
                self.rate.update(len(acc) - 1, min_len)
            self.accepted_draft_tokens += len(acc) - 1
            self.drafted_tokens += min_len
            self.seqs[j].extend(acc)                                    # kv_pos moves by len(acc): later positions are overwritten
            out.append(acc)
        return out, (logits.reshape(bsz, q_len, -1) if logits is not None else None)
