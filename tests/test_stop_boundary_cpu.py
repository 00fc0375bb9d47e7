"""Stop boundaries: where the scanner allows a stop, where it refuses, and how a token stream defers."""
from ninfer_fusion_b200.frontend.stop_boundary import (CODE_BLOCK_CLOSE, CODE_STATEMENT, FENCE_CLOSE, NONE, PARAGRAPH,
                                                       PROSE_SENTENCE, BoundaryScanner, StopPolicy, pause_notice)


def classes(text, policy=None):
    """The boundary class after each line end of `text`, fed one character per token."""
    s = BoundaryScanner(policy)
    out = []
    for ch in text:
        d = s.observe_token(ch)
        if ch == "\n":
            out.append(d.boundary)
    return out, s


def test_code_inside_a_fence():
    text = ("```c\n"
            "int f(int a) {\n"
            "    int x = g(\n"
            "        a);\n"
            "    if (x)\n"
            "        return 1;\n"
            "    // done; }\n"
            "    /* block;\n"
            "       still; */\n"
            "    char* s = \"semi;\n"
            "    return 0; /* tail */\n"
            "}\n"
            "```\n")
    got, s = classes(text)
    assert got == [NONE,               # the fence opener
                   NONE,               # '{' opens a block
                   NONE,               # '(' still open at the line end
                   CODE_STATEMENT,     # ');' closes the call: the statement is complete
                   NONE,               # 'if (x)': the statement continues on the next line
                   CODE_STATEMENT,
                   NONE,               # a comment-only line is not vouched for
                   NONE, NONE,         # inside / closing a block comment
                   NONE,               # an unterminated string: nothing is claimed
                   CODE_STATEMENT,     # the comment after ';' is not content
                   CODE_BLOCK_CLOSE,
                   FENCE_CLOSE]
    assert not s.in_fence and s.paren == 0 and s.brace == 0


def test_strings_triple_quotes_and_continuations():
    text = ("```python\n"
            "x = \"a;\"\n"             # ends in a quote: terminates nothing
            "y = '''one;\n"
            "two;\n"
            "'''\n"
            "z = 1 + \\\n"
            "    2;\n"
            "s = \"\";\n"              # an empty string is not the start of a tripled one
            "# comment;\n"
            "t = f(\"}\");\n"
            "```\n")
    got, _ = classes(text)
    assert got == [NONE, NONE, NONE, NONE, NONE, NONE, CODE_STATEMENT, CODE_STATEMENT, NONE, CODE_STATEMENT, FENCE_CLOSE]


def test_prose_paragraphs_sentences_and_policy():
    text = "It's done.\nSee (fig.\n1) now.\n\nA list:\n- item :(\n\nNext e.g.\n"
    got, _ = classes(text)
    assert got == [PROSE_SENTENCE,     # the apostrophe is not a string in prose
                   NONE,               # '(' open across the line end
                   PROSE_SENTENCE,
                   PARAGRAPH,
                   NONE,
                   NONE,               # ':(' leaves a '(' open ...
                   NONE,               # ... so even the blank line is refused, but the paragraph resets the count
                   PROSE_SENTENCE]
    strict, _ = classes("Done.\n\nNext.\n", StopPolicy(prose_sentence_is_boundary=False, paragraph_is_boundary=False))
    assert strict == [NONE, NONE, NONE]
    code_like, _ = classes("call();\n}\nuse `a;\nb`.\nok.\n")
    # an inline span does not cross lines: the stray back-tick of the fourth line opens a new span (nothing is claimed
    # for that line) which ends with the line
    assert code_like == [CODE_STATEMENT, CODE_BLOCK_CLOSE, NONE, NONE, PROSE_SENTENCE]


def test_a_token_stream_defers_until_the_boundary_and_reports_overrun():
    s = BoundaryScanner(StopPolicy(deferral_report_tokens=3))
    pieces = ["```", "js", "\n", "let", " a", " =", " [", "1", ",", "\n", " 2", "]", ";", "\n", "```", "\n", "Done", "."]
    safe_at = [i for i, p in enumerate(pieces) if s.observe_token(p).safe]
    assert safe_at == [13, 15]                       # after '];\n' and after the closing fence; never inside the array
    d = s.decision()
    assert not d.safe and d.tokens_since_boundary == 2 and not d.deferral_overran
    for p in [" and", " so", " on"]:
        d = s.observe_token(p)
    assert d.deferral_overran and not d.safe          # the bound reports, it does not license a stop
    n = pause_notice(d, "soft_max_tokens")
    assert n["state"] == "deferred" and n["emits_tokens"] is False and n["boundary"] == NONE
    d = s.observe_token("!\n")
    assert d.safe and d.boundary == PROSE_SENTENCE and pause_notice(d, "x")["state"] == "stopped"
    assert s.observe_token(" ").safe is False         # one more character: the output no longer ends at the boundary


def test_soft_max_tokens_ends_a_generation_at_the_next_safe_boundary():
    """The service cancels a generation that has passed its soft limit as soon as the text ends at a boundary; the
    notice travels beside the text; with no boundary before the hard limit the notice says 'deferred'."""
    from ninfer_fusion_b200 import cli
    from ninfer_fusion_b200.frontend.tokenizer import Tokenizer
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.engine import Engine
    from ninfer_fusion_b200.runtime.program import ReferenceProgram
    from ninfer_fusion_b200.serve import protocols as P
    from ninfer_fusion_b200.serve.service import GenerationService, GenRequest
    tok = Tokenizer.train_toy(cli.DEFAULT_CORPUS, 200, cli.SPECIAL_TOKENS)
    text = "```c\nint a = f(\n  1);\nint b = 2;\n```\nAll done.\nmore words follow here and go on"
    script = tok.encode(text)

    class Scripted(ReferenceProgram):
        """Emits the script's tokens one after the other, whatever the model computes."""

        def prefill_step(self, lane, budget):
            first = super().prefill_step(lane, budget)
            if first is not None:
                lane.script_at = 1
                lane.last_token = script[0]
                return script[0]
            return None

        def decode_round(self, lanes):
            out = []
            for lane in lanes:
                super().decode_round([lane])
                lane.last_token = script[min(lane.script_at, len(script) - 1)]
                lane.script_at += 1
                out.append(lane.last_token)
            return out

    cfg = TINY_DENSE.shrink(2)
    w = random_weights(cfg, "cpu", seed=5, std=0.05)
    eng = Engine(lambda: Scripted(cfg, w, max_lanes=2, max_context=512), prefill_chunk=32)
    svc = GenerationService(eng, tok, "scripted", max_concurrent=2, queue_timeout_s=20.0)
    try:
        inside = len(tok.encode("```c\nint a = f(\n"))          # the soft limit falls inside the open call
        res = svc.generate(GenRequest(prompt="go", max_tokens=len(script), soft_max_tokens=inside, enable_thinking=False))
        assert res.content == "```c\nint a = f(\n  1);\n" and res.finish_reason == "length"
        assert res.stop_boundary["state"] == "stopped" and res.stop_boundary["boundary"] == CODE_STATEMENT
        assert res.stop_boundary["reason"] == "soft_max_tokens" and res.stop_boundary["emits_tokens"] is False
        body = P.openai_chat_response(res, "m")
        assert body["stop_boundary"]["boundary"] == CODE_STATEMENT and body["choices"][0]["finish_reason"] == "length"
        # the hard limit first: nothing is cut short, the notice says how far from a boundary the text ends
        hard = len(tok.encode("```c\nint a = f(\n  1"))
        res = svc.generate(GenRequest(prompt="go", max_tokens=hard, soft_max_tokens=hard, enable_thinking=False))
        assert res.finish_reason == "length" and res.stop_boundary["state"] == "deferred" and res.stop_boundary["paren_depth"] == 1
        # without the field nothing changes
        res = svc.generate(GenRequest(prompt="go", max_tokens=12, enable_thinking=False))
        assert res.stop_boundary is None and res.completion_tokens == 12
    finally:
        eng.shutdown()
    req, _ = P.parse_openai_chat({"messages": [{"role": "user", "content": "x"}], "max_tokens": 64, "soft_max_tokens": 48})
    assert req.soft_max_tokens == 48
    req, _ = P.parse_anthropic_messages({"messages": [{"role": "user", "content": "x"}], "max_tokens": 64, "soft_max_tokens": 8})
    assert req.soft_max_tokens == 8
    req, _ = P.parse_openai_responses({"input": "x", "max_output_tokens": 64, "soft_max_output_tokens": 32})
    assert req.soft_max_tokens == 32
    import pytest
    for bad in (0, -3, "7", True, 65):
        with pytest.raises(P.BadRequest):
            P.parse_openai_chat({"messages": [{"role": "user", "content": "x"}], "max_tokens": 64, "soft_max_tokens": bad})
