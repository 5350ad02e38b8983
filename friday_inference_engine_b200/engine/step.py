"""The step function: a batch of sequences, each with its next tokens, run as ONE batch
from the cache; logits come back for the places that were asked for.

A step is either the start of sequences (whole prompts of unequal lengths, or any
number of further tokens for sequences that already hold some) or one token for each:
the same code runs both, because every row of the batch carries its own sequence and
position and the kernels read only that.  Rows are the tokens of all sequences laid
end to end, as the reference lays a prompt's tokens out as [T][.] rows
(transformer.cpp:1129-1149); there are no padding rows in a pass, so padding cannot
change a result.

Long inputs are cut into passes of at most `chunk` tokens per sequence (the reference
cuts prompts at 512: transformer.cpp:1369).  A pass runs all layers; the next pass finds
the earlier tokens in the cache.  The cut changes no result beyond rounding.

Host-side layout of a pass (int32, sent to the device in one copy):
    tokens[rows] | row_seq[rows] | row_pos[rows] | want_rows[n] | seq_start[n_seqs] | seq_qlen[n_seqs] |
    seq_pos0[n_seqs] | per group: table[n_seqs][width]
"""
import numpy as np
import torch


class StepError(ValueError):
    """A step that cannot be run: unknown token id, a sequence too long, a bad request."""


class StepContext:
    """The geometry of one pass; parts read it, nothing writes it after it is built."""

    def __init__(self, stepper, slots, q_lens, kv_lens):
        self._stepper = stepper
        self.slots = list(slots)                 # host: cache slot of every sequence
        self.q_lens = list(q_lens)               # host: tokens of this pass per sequence
        self.kv_lens = list(kv_lens)             # host: tokens held after this pass
        self.n_seqs = len(self.slots)
        self.rows = int(sum(self.q_lens))
        self.max_q_len = max(self.q_lens) if self.q_lens else 0
        self.max_kv_len = max(self.kv_lens) if self.kv_lens else 0
        self.decode = self.max_q_len == 1
        self.tokens = self.row_seq = self.row_pos = self.want_rows = self.seq_slots = None
        self.seq_start = self.seq_qlen = self.seq_pos0 = None    # int32 [n_seqs] on the device
        self.tables = []

    def scratch(self, n_floats, device):
        return self._stepper.scratch(n_floats, device)


def _pad4(n):
    return (n + 3) & ~3


class Stepper:
    def __init__(self, model, cache, chunk=2048):
        self.model, self.cache = model, cache
        self.device = model.env.device
        self.chunk = int(chunk)
        self.vocab = model.spec.vocab_size
        self._scratch = None
        self._staging = []            # pinned host buffers with the event of their last copy
        self._next_staging = 0
        self.last_upload_bytes = 0

    def scratch(self, n_floats, device):
        if self._scratch is None or self._scratch.numel() < n_floats:
            self._scratch = torch.empty((max(int(n_floats), 1 << 16),), dtype=torch.float32, device=device)
        return self._scratch

    # -- host to device ----------------------------------------------------
    def _upload(self, host):
        """One copy of a packed int32 array to the device, through pinned memory."""
        n = host.size
        self.last_upload_bytes = 4 * n
        if self.device.type != "cuda":
            return torch.from_numpy(host.copy())
        if len(self._staging) < 4:
            self._staging.append([torch.empty((max(n, 4096),), dtype=torch.int32).pin_memory(), None])
        slot = self._staging[self._next_staging % len(self._staging)]
        self._next_staging += 1
        if slot[1] is not None:
            slot[1].synchronize()              # the copy that last used this buffer is done
        if slot[0].numel() < n:
            slot[0] = torch.empty((n,), dtype=torch.int32).pin_memory()
        slot[0][:n].numpy()[:] = host
        dev = torch.empty((n,), dtype=torch.int32, device=self.device)
        dev.copy_(slot[0][:n], non_blocking=True)
        slot[1] = torch.cuda.Event()
        slot[1].record()
        return dev

    def build_context(self, slots, pass_tokens, want_rows):
        """Reserves pages, packs the pass's numbers, sends them, returns the context."""
        cache = self.cache
        q_lens = [len(t) for t in pass_tokens]
        start = [cache.lens[s] for s in slots]
        cache.reserve(slots, q_lens)
        ctx = StepContext(self, slots, q_lens, [a + q for a, q in zip(start, q_lens)])
        rows = ctx.rows
        tables = cache.tables_for(slots)
        nseq = len(slots)
        sizes = [rows, rows, rows, len(want_rows), nseq, nseq, nseq] + [t.size for t in tables]
        offs = np.concatenate([[0], np.cumsum([_pad4(s) for s in sizes])]).astype(np.int64)
        host = np.zeros((int(offs[-1]),), dtype=np.int32)
        host[offs[0]:offs[0] + rows] = np.concatenate([np.asarray(t, dtype=np.int32) for t in pass_tokens])
        host[offs[1]:offs[1] + rows] = np.repeat(np.arange(len(slots), dtype=np.int32), q_lens)
        host[offs[2]:offs[2] + rows] = np.concatenate(
            [np.arange(a, a + q, dtype=np.int32) for a, q in zip(start, q_lens)])
        host[offs[3]:offs[3] + len(want_rows)] = np.asarray(want_rows, dtype=np.int32)
        host[offs[4]:offs[4] + nseq] = np.concatenate([[0], np.cumsum(q_lens)[:-1]]).astype(np.int32)
        host[offs[5]:offs[5] + nseq] = np.asarray(q_lens, dtype=np.int32)
        host[offs[6]:offs[6] + nseq] = np.asarray(start, dtype=np.int32)
        for i, t in enumerate(tables):
            host[offs[7 + i]:offs[7 + i] + t.size] = t.reshape(-1)
        dev = self._upload(host)
        ctx.tokens = dev[offs[0]:offs[0] + rows]
        ctx.row_seq = dev[offs[1]:offs[1] + rows]
        ctx.row_pos = dev[offs[2]:offs[2] + rows]
        ctx.want_rows = dev[offs[3]:offs[3] + len(want_rows)]
        ctx.seq_start = dev[offs[4]:offs[4] + nseq]
        ctx.seq_qlen = dev[offs[5]:offs[5] + nseq]
        ctx.seq_pos0 = dev[offs[6]:offs[6] + nseq]
        ctx.tables = [dev[offs[7 + i]:offs[7 + i] + t.size].view(t.shape) for i, t in enumerate(tables)]
        ctx.seq_slots = torch.as_tensor(slots, dtype=torch.int64, device=self.device) if cache.states else None
        return ctx

    def views(self, ctx):
        return [None if call.cache is None
                else self.cache.view(call.cache, call.write, ctx.tables, ctx.seq_slots, ctx.slots)
                for call in self.model.program]

    # -- the step ------------------------------------------------------------
    def check(self, slots, tokens, want):
        if not slots:
            raise StepError("a step needs at least one sequence")
        if len(set(slots)) != len(slots):
            raise StepError("a sequence appears twice in one step")
        if not (len(tokens) == len(slots) == len(want)):
            raise StepError("slots, tokens and want must have one item per sequence")
        limit = min(self.cache.max_seq_tokens, self.model.spec.max_positions)
        for slot, toks, w in zip(slots, tokens, want):
            if len(toks) == 0:
                raise StepError("a sequence in a step brings no token")
            lo, hi = min(toks), max(toks)
            if lo < 0 or hi >= self.vocab:
                raise StepError("token id %d is outside the vocabulary [0, %d)" % (lo if lo < 0 else hi, self.vocab))
            if self.cache.lens[slot] + len(toks) > limit:
                raise StepError("context length exceeded: the sequence would hold %d tokens, the limit is %d"
                                % (self.cache.lens[slot] + len(toks), limit))
            for p in w:
                if not 0 <= p < len(toks):
                    raise StepError("logits wanted at place %d of %d tokens" % (p, len(toks)))

    def step(self, slots, tokens, want):
        """slots: cache slots, one per sequence; tokens: for each its next token ids;
        want: for each the places among these tokens whose logits are asked for.
        Returns fp32 logits [sum(len(w) for w in want), vocab] on the device, in the order
        of the sequences and, within one, of `want`."""
        self.check(slots, tokens, want)
        n = len(slots)
        done = [0] * n
        pieces, order = [], []          # logits of each pass; (sequence, index in want) of their rows
        while True:
            live = [i for i in range(n) if done[i] < len(tokens[i])]
            if not live:
                break
            pass_tokens = [tokens[i][done[i]:done[i] + self.chunk] for i in live]
            want_rows, base = [], 0
            for i, pt in zip(live, pass_tokens):
                for wi, p in enumerate(want[i]):
                    if done[i] <= p < done[i] + len(pt):
                        want_rows.append(base + p - done[i])
                        order.append((i, wi))
                base += len(pt)
            pass_slots = [slots[i] for i in live]
            ctx = self.build_context(pass_slots, pass_tokens, want_rows)
            x = self.model.run(ctx.tokens, ctx, self.views(ctx))
            if want_rows:
                pieces.append(self.model.logits(x, ctx.want_rows))
            self.cache.commit(pass_slots, ctx.q_lens)
            for i, pt in zip(live, pass_tokens):
                done[i] += len(pt)
        if not pieces:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=self.device)
        out = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)
        wanted = sorted(range(len(order)), key=lambda r: order[r])
        if wanted != list(range(len(order))):
            out = out[torch.as_tensor(wanted, dtype=torch.int64, device=out.device)]
        return out
