"""Token / acceptance parity of a CUDA run against the oracle, cycle by cycle, without giving up at a near-tie.

Test infrastructure (like everything under oracle/): used by tests/, by __graft_entry__.smoke() and by the
cpu_baseline leg of bench.py, never by the product.

The north star's rule: token ids and per-cycle acceptance counts equal the reference's, a divergence being allowed
only where the reference's top-2 logit gap is below 1e-3.  `follow_generation` replays the event on the oracle while
following the CUDA run: every cycle starts from the token the CUDA run emitted last, the oracle samples its own
draft and target tokens, and the cycle's outcome (accepted, committed, emitted tokens) is compared.  Where the two
differ, the first differing decision must be a near-tie in the oracle's own logits (draft logits for a draft token,
target logits for a target token); the oracle then repeats the cycle with the CUDA run's tokens forced, so that
its stream state keeps following the CUDA run and every later cycle is still compared.
"""

from __future__ import annotations

GAP_LIMIT = 1e-3


def follow_generation(oracle, stream, prompt, cuda_tokens, cuda_cycles, drafts, gap_limit=GAP_LIMIT, prefill_chunk=64, max_cycles=None,
                      cycle_seconds=None, seconds_budget=None):
    """Replays `prompt` + the generated `cuda_tokens` on `oracle`/`stream`.

    cuda_cycles: the engine's cycle log (dicts with accepted, committed, emitted, target_token_ids) - empty for a run
    without speculation.  Returns a dict: tokens_compared, cycles_compared, tokens_equal (no divergence at all),
    divergences (list of dicts: position, kind, gap, cuda, oracle), violations (divergences whose gap is not below
    gap_limit: parity failures), accepted_equal (per-cycle acceptance counts equal wherever the tokens were).
    cycle_seconds: optional list that receives the wall time of every (first, unforced) oracle cycle; with
    seconds_budget the replay stops once those add up to it (a bounded sample of a long run).
    """
    import time

    report = {"tokens_compared": 0, "cycles_compared": 0, "tokens_equal": True, "accepted_equal": True, "divergences": [], "violations": []}

    def note(position, kind, gap, cuda, mine):
        entry = {"position": position, "kind": kind, "gap": float(gap), "cuda": int(cuda), "oracle": int(mine)}
        report["tokens_equal"] = False
        report["divergences"].append(entry)
        if not gap < gap_limit:
            report["violations"].append(entry)

    if not cuda_tokens:
        oracle.prefill(stream, prompt, sample_last=False, chunk=prefill_chunk)
        return report
    first, logits = oracle.prefill(stream, prompt, sample_last=True, chunk=prefill_chunk)
    report["tokens_compared"] = 1
    if first != cuda_tokens[0]:
        note(0, "prefill target", oracle.top2_gap(logits[0]), cuda_tokens[0], first)
    position = 1  # tokens of the CUDA run consumed so far
    token = cuda_tokens[0]
    cycle_index = 0
    while position < len(cuda_tokens):
        if max_cycles is not None and report["cycles_compared"] >= max_cycles:
            break
        if seconds_budget is not None and cycle_seconds is not None and sum(cycle_seconds) > seconds_budget:
            break
        remaining = len(cuda_tokens) - position
        if drafts > 0 and oracle.pkg.draft is not None and cycle_index < len(cuda_cycles) and remaining >= 2:
            theirs = cuda_cycles[cycle_index]
            cycle_index += 1
            count = min(drafts, remaining - 1)
            saved = oracle.checkpoint(stream)
            started = time.perf_counter()
            mine = oracle.speculative_cycle(stream, token, count)
            if cycle_seconds is not None:
                cycle_seconds.append(time.perf_counter() - started)
            emitted = [int(t) for t in theirs["emitted"]]
            same = mine["emitted"] == emitted and mine["accepted"] == int(theirs["accepted"])
            if not same:
                # the first decision that differs: a draft token (an accepted draft of the CUDA run is its emitted
                # token; behind the accepted prefix the CUDA run's draft is only known to differ from its target) or a
                # target token
                accepted = int(theirs["accepted"])
                targets = [int(t) for t in theirs["target_token_ids"]]
                explained = False
                for j in range(count + 1):
                    if j < count:
                        cuda_draft = emitted[j] if j < accepted else None
                        if cuda_draft is not None and mine["draft_token_ids"][j] != cuda_draft:
                            note(position + j, "draft", oracle.top2_gap(mine["draft_logits"][j]), cuda_draft, mine["draft_token_ids"][j])
                            explained = True
                            break
                        if cuda_draft is None and j < len(targets) and mine["draft_token_ids"][j] == targets[j] == mine["target_token_ids"][j]:
                            # the oracle accepts draft j, the CUDA run rejected it: its draft differed from this one
                            note(position + j, "draft", oracle.top2_gap(mine["draft_logits"][j]), 0xFFFFFFFF, mine["draft_token_ids"][j])
                            explained = True
                            break
                    if j < len(targets) and mine["target_token_ids"][j] != targets[j]:
                        note(position + j, "target", oracle.top2_gap(mine["target_logits"][j]), targets[j], mine["target_token_ids"][j])
                        explained = True
                        break
                    if j >= accepted:
                        break
                if not explained:
                    note(position, "cycle outcome", float("inf"), accepted, mine["accepted"])
                    report["accepted_equal"] = False
                # follow the CUDA run: the same cycle again with its tokens forced
                oracle.restore(stream, saved)
                forced_drafts = [emitted[j] if j < accepted else ((targets[j] + 1) % oracle.pkg.vocab if j < len(targets) else 0) for j in range(count)]
                redo = oracle.speculative_cycle(stream, token, count, forced_drafts=forced_drafts, forced_targets=targets)
                if redo["emitted"] != emitted:
                    report["accepted_equal"] = False
                    note(position, "forced replay", float("inf"), len(emitted), len(redo["emitted"]))
                    break
            report["cycles_compared"] += 1
            report["tokens_compared"] += len(emitted)
            position += len(emitted)
            token = emitted[-1]
        else:
            saved = oracle.checkpoint(stream)
            mine, logits = oracle.single_tick(stream, token, emit=True)
            theirs = cuda_tokens[position]
            if mine != theirs:
                note(position, "target", oracle.top2_gap(logits[0]), theirs, mine)
            report["tokens_compared"] += 1
            position += 1
            token = theirs
    return report


def summary(report):
    worst = max((d["gap"] for d in report["divergences"]), default=0.0)
    return {"tokens_compared": report["tokens_compared"], "cycles_compared": report["cycles_compared"], "tokens_equal": report["tokens_equal"],
            "accepted_equal": report["accepted_equal"], "divergences": len(report["divergences"]), "violations": len(report["violations"]),
            "largest_gap_at_a_divergence": worst, "gap_limit": GAP_LIMIT}
