"""The generation loop: prompts in, tokens out, for as many requests as there are.

Requests are run in batches of at most `max_batch`, one batch after another.  A batch
starts with all its prompts in one step; then every live sequence takes one token per
step.  A sequence ends when it draws a stop token (which is not kept, as the reference
prints nothing for it: main.cpp:331-332), when it has `max_new_tokens`, or when its
context is full (main.cpp:335); it then leaves the batch, its slot goes back at once,
and the others go on.  A prompt that would fill the context is refused before anything
runs (main.cpp:319-322).

The loop knows no kernels: it is given a step function, a sampler and the slot
bookkeeping, so its decisions can be tested alone.
"""
from dataclasses import dataclass, field


@dataclass
class Generation:
    tokens: list = field(default_factory=list)
    finish_reason: str = ""            # "stop" | "length" | "context"


class GenerationError(ValueError):
    pass


def generate(prompts, *, step, sample, alloc_slot, free_slot, max_batch, max_context, vocab_size,
             max_new_tokens=100, stop_token_ids=(), ignore_eos=False, on_step=None, decoder=None):
    """step(slots, tokens, want) -> logits rows; sample(logits, streams, steps) -> list of ids.

    decoder (optional): decoder(slots, first_tokens, streams, steps_done) -> object with
    step(tokens) -> chosen ids for all its rows, retire(row) and close(); it then runs the
    one-token steps (model, sampler and all) instead of step + sample.  The decisions
    below are the same either way.

    Stream numbers are the positions of the requests in `prompts`, so a request draws the
    same tokens whichever batch it lands in.
    """
    stop = frozenset() if ignore_eos else frozenset(int(t) for t in stop_token_ids)
    prompts = [list(p) for p in prompts]
    for r, p in enumerate(prompts):
        if not p:
            raise GenerationError("request %d has an empty prompt" % r)
        if len(p) >= max_context:
            raise GenerationError("request %d: the prompt (%d tokens) is longer than the context (%d); use --ctx"
                                  % (r, len(p), max_context))
        bad = [t for t in p if not 0 <= t < vocab_size]
        if bad:
            raise GenerationError("request %d: token id %d is outside the vocabulary [0, %d)" % (r, bad[0], vocab_size))
    results = [Generation() for _ in prompts]
    if max_new_tokens <= 0:
        for g in results:
            g.finish_reason = "length"
        return results

    def settle(r, tok):
        """Books token `tok` for request r; True if the request goes on."""
        g = results[r]
        if tok in stop:
            g.finish_reason = "stop"
        else:
            g.tokens.append(tok)
            if len(g.tokens) >= max_new_tokens:
                g.finish_reason = "length"
            elif len(prompts[r]) + len(g.tokens) - 1 >= max_context:
                g.finish_reason = "context"
        return not g.finish_reason

    for first in range(0, len(prompts), max_batch):
        batch = list(range(first, min(first + max_batch, len(prompts))))
        slot_of = {}
        dec = None
        try:
            for r in batch:
                slot_of[r] = alloc_slot()
            live = batch
            logits = step([slot_of[r] for r in live], [prompts[r] for r in live], [[len(prompts[r]) - 1] for r in live])
            drawn = sample(logits, live, [0] * len(live))
            if on_step is not None:
                on_step(live, drawn)
            live = [r for r, tok in zip(live, drawn) if settle(r, tok) or free_slot(slot_of.pop(r))]
            if decoder is not None and live:
                rows = list(live)                      # row i of the decoder belongs to request rows[i], for good
                dec = decoder([slot_of[r] for r in rows], [results[r].tokens[-1] for r in rows], rows,
                              [len(results[r].tokens) for r in rows])
                while live:
                    drawn_rows = dec.step([results[r].tokens[-1] if r in slot_of else 0 for r in rows])
                    if on_step is not None:
                        on_step(live, [drawn_rows[rows.index(r)] for r in live])
                    for r in list(live):
                        if not settle(r, drawn_rows[rows.index(r)]):
                            dec.retire(rows.index(r))
                            free_slot(slot_of.pop(r))
                            live.remove(r)
            while live:
                logits = step([slot_of[r] for r in live], [[results[r].tokens[-1]] for r in live], [[0]] * len(live))
                drawn = sample(logits, live, [len(results[r].tokens) for r in live])
                if on_step is not None:
                    on_step(live, drawn)
                live = [r for r, tok in zip(live, drawn) if settle(r, tok) or free_slot(slot_of.pop(r))]
        finally:
            if dec is not None:
                dec.close()
            for s in slot_of.values():          # an error in the middle gives the slots back too
                free_slot(s)
    return results
