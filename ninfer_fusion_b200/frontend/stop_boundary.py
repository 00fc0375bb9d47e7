"""Where generation may be interrupted: a scanner for syntax-safe stop boundaries.

A generation that is cut by a budget (or paused so that something can be recalled) should not end in the middle of a
string, an expression or a half-written statement.  The scanner reads the decoded text of the committed tokens, in
order, and answers one question: "is the current end of the output a legal place to stop?"  It reads the SURFACE text,
not token ids, because a byte-level BPE token is not a lexeme (`";` and `}\\n` are single tokens).

Boundary classes (a line end is judged by the line's last significant character):

* `code-statement`    the line ends in `;`
* `code-block-close`  the line ends in `}`
* `fence-close`       the line closes a ``` / ~~~ fence
* `paragraph`         a blank line
* `prose-sentence`    the line ends in a sentence terminator (. ! ? and the full-width forms); optional by policy,
                      since "e.g." at a line end is the one realistic false positive

Never a boundary: a line end while a `(` or `[` is open (the expression continues), inside a string, a triple-quoted
string, a block comment or after a backslash continuation; a line that ends in `)`, `{`, `,` or an operator; a line
that is only a comment (the scanner does not read comments as content and will not vouch for what it has not read).
Brace depth does not disqualify: a statement inside a function body is a complete statement.  Inside a fenced code
block only the code classes and the fence close count; outside a fence only the prose classes, the fence close, and the
code classes when the line looks like code (ends in `;` or `}`).

The scanner keeps a few counters and characters, never the whole output.  A deferral bound is a REPORTING bound: when
more than `deferral_report_tokens` tokens pass without a boundary the decision says so, and stopping is still refused.

Reference: src/spec/stop_boundary.h (the classes, what is deliberately not a boundary, the check-then-commit contract,
the out-of-band pause notice).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

NONE = "none"
CODE_STATEMENT = "code-statement"
CODE_BLOCK_CLOSE = "code-block-close"
FENCE_CLOSE = "fence-close"
PARAGRAPH = "paragraph"
PROSE_SENTENCE = "prose-sentence"
SENTENCE_END = ".!?。！？"


@dataclass(frozen=True)
class StopPolicy:
    prose_sentence_is_boundary: bool = True
    paragraph_is_boundary: bool = True
    deferral_report_tokens: int = 64


@dataclass
class StopDecision:
    safe: bool = False
    boundary: str = NONE
    tokens_since_boundary: int = 0
    deferral_overran: bool = False
    in_string: bool = False
    in_block_comment: bool = False
    in_fence: bool = False
    paren_depth: int = 0
    brace_depth: int = 0
    tokens_seen: int = 0


class BoundaryScanner:
    def __init__(self, policy: Optional[StopPolicy] = None):
        self.policy = policy or StopPolicy()
        self.tokens_seen = 0
        self.tokens_since_boundary = 0
        self.paren = 0                   # '(' and '[' nesting
        self.brace = 0
        self.string = ""                 # "", one of " ' ` , or a tripled quote
        self.escape = False
        self.block_comment = False
        self.line_comment = False
        self.in_fence = False
        self.fence_mark = ""
        self.last_line_class = NONE
        self._at_boundary = NONE         # class of the boundary the output currently ends at
        self._head = ""                  # first characters of the current line (fence detection)
        self._last_sig = ""              # last significant character of the line (outside strings and comments)
        self._has_content = False        # the line has something besides white space and comments
        self._has_comment = False
        self._continued = False          # the last significant thing on the line is a backslash
        self._p1 = ""                    # previous character
        self._just_opened = False        # the string was opened by the previous character
        self._empty_pair = ""            # an empty string "" / '' closed at the previous character
        self._quote_run = 0              # consecutive quote characters inside a tripled string
        self._blank_run = 0              # consecutive line ends

    # ------------------------------------------------------------------ feeding
    def observe_token(self, text: str) -> StopDecision:
        """The decoded text of ONE committed token (may be empty: bytes that complete a later character)."""
        self.tokens_seen += 1
        self.tokens_since_boundary += 1
        for ch in text:
            self._char(ch)
        if self._at_boundary != NONE:
            self.tokens_since_boundary = 0
        return self.decision()

    def decision(self) -> StopDecision:
        b = self._at_boundary
        return StopDecision(b != NONE, b, self.tokens_since_boundary,
                            self.tokens_since_boundary > self.policy.deferral_report_tokens, bool(self.string),
                            self.block_comment, self.in_fence, self.paren, self.brace, self.tokens_seen)

    # ------------------------------------------------------------------ the state machine
    def _is_fence_line(self) -> bool:
        lead = len(self._head) - len(self._head.lstrip(" "))
        return lead <= 3 and self._head[lead:lead + 3] in ("```", "~~~")

    def _char(self, ch: str) -> None:
        if ch == "\r":
            return
        if ch == "\n":
            self._end_line()
            self._p1 = ch
            return
        self._at_boundary = NONE          # anything after the line end: the output no longer ends at the boundary
        self._blank_run = 0 if ch not in " \t" else self._blank_run
        if len(self._head) < 8:
            self._head += ch
        p1, self._p1 = self._p1, ch
        if self.line_comment:
            return
        if self.block_comment:
            if p1 == "*" and ch == "/":
                self.block_comment = False
                self._p1 = ""             # the '/' that closed the comment does not open the next one
            return
        if self.string:
            self._string_char(ch)
            return
        if ch in " \t":
            self._empty_pair = ""
            return
        if self._is_fence_line():          # a fence marker line is neither code nor prose
            self._has_content = True
            return
        code = self.in_fence
        empty_pair, self._empty_pair = self._empty_pair, ""
        self._continued = False
        if code and ch == "/" and p1 == "/":
            self.line_comment = self._has_comment = True
            self._retract("/")
        elif code and ch == "*" and p1 == "/":
            self.block_comment = self._has_comment = True
            self._retract("/")
        elif code and ch == "#" and not self._has_content:
            self.line_comment = self._has_comment = True
        elif ch == "`" or (code and ch in "\"'"):
            if empty_pair == ch:
                self.string, self._quote_run = ch * 3, 0      # the third quote in a row opens a tripled string
            else:
                self.string, self._just_opened = ch, True
            self._has_content, self._last_sig = True, ch
        else:
            if ch == "\\":
                self._continued = True
            elif ch in "([":
                self.paren += 1
            elif ch in ")]":
                self.paren = max(0, self.paren - 1)
            elif ch == "{":
                self.brace += 1
            elif ch == "}":
                self.brace = max(0, self.brace - 1)
            self._prev_sig, self._prev_content = self._last_sig, self._has_content
            self._has_content, self._last_sig = True, ch

    _prev_sig, _prev_content = "", False

    def _retract(self, ch: str) -> None:
        """The first character of a comment opener was taken as content before the opener was recognised."""
        if self._last_sig == ch:
            self._last_sig, self._has_content = self._prev_sig, self._prev_content

    def _string_char(self, ch: str) -> None:
        opened, self._just_opened = self._just_opened, False
        if self.escape:
            self.escape = False
            return
        if ch == "\\":
            self.escape = True
            self._quote_run = 0
            return
        q = self.string
        if len(q) == 3:
            self._quote_run = self._quote_run + 1 if ch == q[0] else 0
            if self._quote_run == 3:
                self.string, self._last_sig = "", ch
        elif ch == q:
            self.string, self._last_sig = "", ch
            if opened and ch != "`":
                self._empty_pair = ch       # "" so far: one more quote makes it a tripled string

    def _end_line(self) -> None:
        cls = NONE
        self._blank_run += 1
        tripled = len(self.string) == 3
        if self.block_comment or tripled or self._continued:
            pass                              # the unit continues on the next line
        elif self._is_fence_line():
            lead = self._head.lstrip(" ")
            mark = lead[:3]
            if self.in_fence:
                if mark == self.fence_mark and lead.strip(mark[0] + " \t") == "":
                    self.in_fence, self.fence_mark = False, ""
                    self.paren = self.brace = 0       # what the block left open does not leak into the prose
                    cls = FENCE_CLOSE
            else:
                self.in_fence, self.fence_mark = True, mark
        elif self.string:
            pass                              # an unterminated one-line string: no boundary is claimed for this line
        elif not self._has_content:
            if not self._has_comment and not self.in_fence:
                if self.policy.paragraph_is_boundary and self.paren == 0 and self._blank_run >= 2:
                    cls = PARAGRAPH
                if self._blank_run >= 2:
                    self.paren = 0            # prose: a stray "(" (an emoticon, a list marker) ends with its paragraph
        elif self.paren == 0:
            last = self._last_sig
            if last == ";":
                cls = CODE_STATEMENT
            elif last == "}":
                cls = CODE_BLOCK_CLOSE
            elif last and last in SENTENCE_END and not self.in_fence and self.policy.prose_sentence_is_boundary:
                cls = PROSE_SENTENCE
        if len(self.string) == 1:
            self.string = ""                  # one-line strings and inline code spans end with their line
        self.last_line_class = self._at_boundary = cls
        self.line_comment = self.escape = False
        self._head, self._last_sig = "", ""
        self._has_content = self._has_comment = self._continued = self._just_opened = False
        self._empty_pair = ""
        self._prev_sig, self._prev_content = "", False


def pause_notice(decision: StopDecision, reason: str) -> dict:
    """What the caller is told out of band when a stop was taken (or is still being deferred).  It carries no token:
    a pause is never written into the generated stream."""
    return {"state": "stopped" if decision.safe else "deferred", "reason": reason, "boundary": decision.boundary,
            "tokens_since_boundary": decision.tokens_since_boundary, "deferral_overran": decision.deferral_overran,
            "in_string": decision.in_string, "in_block_comment": decision.in_block_comment, "in_fence": decision.in_fence,
            "paren_depth": decision.paren_depth, "emits_tokens": False}
