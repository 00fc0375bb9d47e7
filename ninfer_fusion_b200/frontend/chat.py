"""Chat-template rendering and incremental output parsing for the Qwen3.x family.

The template is implemented natively (no Jinja interpreter at run time), as the reference does: a renderer is
selected by the SHA-256 of the artifact's `chat_template.jinja` resource and an unknown template is refused
rather than guessed (src/targets/qwen3_6/impl/frontend/chat_template.cpp:430).  The output side splits the
generated text into reasoning (`<think>` frame), visible content and tool calls (`<tool_call>` JSON frames) while
it streams (src/targets/qwen3_6/impl/frontend/frontend.cpp: thinking / stop / tool-call session).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

IM_START, IM_END = "<|im_start|>", "<|im_end|>"
TOOLS_HEADER = ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
                "You are provided with function signatures within <tools></tools> XML tags:\n<tools>")
TOOLS_FOOTER = ("\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
                "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": "
                "<args-json-object>}\n</tool_call>")

# sha256(chat_template.jinja) -> renderer name.  Artifacts written by this package embed the marker template below.
BUILTIN_TEMPLATE = "{# ninfer-fusion-b200 native chat template: qwen3-hybrid-v1 #}\n"
KNOWN_TEMPLATES: Dict[str, str] = {hashlib.sha256(BUILTIN_TEMPLATE.encode()).hexdigest(): "qwen3"}


class TemplateRefused(ValueError):
    pass


def renderer_for(template_text: Optional[str], allow_unknown: bool = False) -> str:
    if template_text is None:
        return "qwen3"
    digest = hashlib.sha256(template_text.encode("utf-8")).hexdigest()
    name = KNOWN_TEMPLATES.get(digest)
    if name is None:
        if allow_unknown:
            return "qwen3"
        raise TemplateRefused(f"chat template {digest[:16]}… is not one of the compiled renderers; refusing to guess")
    return name


IMAGE_PLACEHOLDER = "<|vision_start|><|image_pad|><|vision_end|>"
VIDEO_PLACEHOLDER = "<|vision_start|><|video_pad|><|vision_end|>"


def _parts_of(content) -> List[Tuple[str, bool]]:
    """OpenAI-style content (a string or a list of typed parts) as (text, is_literal) fragments: text parts are the
    caller's literal text, media parts become the template's own placeholder."""
    if content is None:
        return []
    if isinstance(content, str):
        return [(content, True)]
    out: List[Tuple[str, bool]] = []
    for part in content:
        if isinstance(part, str):
            out.append((part, True))
        elif part.get("type") in ("text", "input_text", "output_text"):
            out.append((part.get("text", ""), True))
        elif part.get("type") in ("image_url", "image", "input_image"):
            out.append((IMAGE_PLACEHOLDER, False))
        elif part.get("type") in ("video_url", "video"):
            out.append((VIDEO_PLACEHOLDER, False))
    return out


def _text_of(content) -> str:
    return "".join(t for t, _ in _parts_of(content))


class _Fragments:
    """The rendered prompt as it is built: text plus the character spans that are the caller's literal text.  What
    the template writes may carry control tokens; what the caller wrote may not (the tokenizer reads the spans)."""

    def __init__(self) -> None:
        self.parts: List[str] = []
        self.spans: List[Tuple[int, int]] = []
        self.n = 0

    def template(self, text: str) -> None:
        if text:
            self.parts.append(text)
            self.n += len(text)

    def literal(self, text: str) -> None:
        if text:
            if self.spans and self.spans[-1][1] == self.n:
                self.spans[-1] = (self.spans[-1][0], self.n + len(text))
            else:
                self.spans.append((self.n, self.n + len(text)))
            self.parts.append(text)
            self.n += len(text)

    def content(self, content) -> None:
        for text, lit in _parts_of(content):
            (self.literal if lit else self.template)(text)


def render_chat_spans(messages: Sequence[dict], tools: Optional[Sequence[dict]] = None, add_generation_prompt: bool = True,
                      enable_thinking: bool = True) -> Tuple[str, List[Tuple[int, int]]]:
    """The rendered prompt and the character spans [begin, end) of it that came from the caller: message contents,
    earlier reasoning, tool-call arguments, tool results and tool schemas.  Everything else is the template.
    Reference: src/spec/frame_axis.h (the template / literal origin of every prompt position, kept as a column),
    src/targets/qwen3_6/impl/frontend/chat_template.cpp (literal spans recorded while rendering)."""
    msgs = list(messages)
    f = _Fragments()
    system = None
    if msgs and msgs[0].get("role") in ("system", "developer"):
        system = msgs[0].get("content")
        msgs = msgs[1:]
    has_system = bool(_text_of(system))
    if tools:
        f.template(f"{IM_START}system\n")
        if has_system:
            f.content(system)
            f.template("\n\n")
        f.template(TOOLS_HEADER)
        for t in tools:
            f.template("\n")
            f.literal(json.dumps(t, ensure_ascii=False))
        f.template(f"{TOOLS_FOOTER}{IM_END}\n")
    elif has_system:
        f.template(f"{IM_START}system\n")
        f.content(system)
        f.template(f"{IM_END}\n")
    # reasoning of earlier turns is dropped; only turns after the last real user query keep it
    last_query = -1
    for i, m in enumerate(msgs):
        if m.get("role") == "user":
            last_query = i
    i = 0
    while i < len(msgs):
        m = msgs[i]
        role = m.get("role")
        if role in ("user", "system", "developer"):
            f.template(f"{IM_START}{'system' if role != 'user' else 'user'}\n")
            f.content(m.get("content"))
            f.template(f"{IM_END}\n")
        elif role == "assistant":
            content = _text_of(m.get("content"))
            reasoning = m.get("reasoning_content") or ""
            if not reasoning and "</think>" in content:
                head, _, content = content.partition("</think>")
                reasoning = head.split("<think>")[-1].strip("\n")
                content = content.lstrip("\n")
            f.template(f"{IM_START}assistant\n")
            if reasoning and i > last_query:
                f.template("<think>\n")
                f.literal(reasoning.strip())
                f.template("\n</think>\n\n")
            if content == _text_of(m.get("content")):
                f.content(m.get("content"))        # untouched by the reasoning split: media parts stay the template's
            else:
                f.literal(content)
            for k, call in enumerate(m.get("tool_calls") or []):
                fn = call.get("function", call)
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except json.JSONDecodeError:
                        pass
                if content or k > 0:
                    f.template("\n")
                f.template("<tool_call>\n")
                f.literal(json.dumps({"name": fn.get("name"), "arguments": args}, ensure_ascii=False))
                f.template("\n</tool_call>")
            f.template(f"{IM_END}\n")
        elif role == "tool":
            # consecutive tool results share one user frame
            f.template(f"{IM_START}user")
            while i < len(msgs) and msgs[i].get("role") == "tool":
                f.template("\n<tool_response>\n")
                f.content(msgs[i].get("content"))
                f.template("\n</tool_response>")
                i += 1
            f.template(f"{IM_END}\n")
            continue
        else:
            raise ValueError(f"unknown message role '{role}'")
        i += 1
    if add_generation_prompt:
        f.template(f"{IM_START}assistant\n")
        if not enable_thinking:
            f.template("<think>\n\n</think>\n\n")
    return "".join(f.parts), f.spans


def render_chat(messages: Sequence[dict], tools: Optional[Sequence[dict]] = None, add_generation_prompt: bool = True,
                enable_thinking: bool = True) -> str:
    """messages: [{"role", "content", optional "reasoning_content", "tool_calls", "tool_call_id"}]."""
    return render_chat_spans(messages, tools, add_generation_prompt, enable_thinking)[0]


# ---------------------------------------------------------------------------------------------------------
# Incremental output parsing
# ---------------------------------------------------------------------------------------------------------
@dataclass
class ToolCall:
    name: str
    arguments: str        # JSON text of the arguments object
    raw: str = ""


@dataclass
class ParsedDelta:
    reasoning: str = ""
    content: str = ""
    tool_calls: List[ToolCall] = field(default_factory=list)


class OutputParser:
    """Feeds on decoded text fragments and separates reasoning / content / tool calls as they stream.

    `thinking=True` means the generation prompt left the model inside an open reasoning frame (the Qwen3 prompt
    does not emit `<think>` itself when thinking is enabled by default in newer templates; an explicit `<think>`
    at the start is accepted too).  Text that could be the beginning of a tag is held back until it is
    disambiguated, so a client never sees half a tag."""

    TAGS = ("<think>", "</think>", "<tool_call>", "</tool_call>")

    def __init__(self, thinking: bool = False, stop: Sequence[str] = ()):
        self.mode = "reasoning" if thinking else "content"
        self.stop = [s for s in stop if s]
        self.stopped = False
        self._hold = ""
        self._tool = ""
        self.reasoning = ""
        self.content = ""
        self.tool_calls: List[ToolCall] = []

    def _emit(self, delta: ParsedDelta, text: str) -> None:
        if not text:
            return
        if self.mode == "reasoning":
            delta.reasoning += text
            self.reasoning += text
        elif self.mode == "tool":
            self._tool += text
        else:
            delta.content += text
            self.content += text

    def _close_tool(self, delta: ParsedDelta) -> None:
        raw = self._tool.strip()
        self._tool = ""
        try:
            obj = json.loads(raw)
            args = obj.get("arguments", {})
            call = ToolCall(str(obj.get("name", "")), args if isinstance(args, str) else json.dumps(args, ensure_ascii=False), raw)
        except (json.JSONDecodeError, AttributeError):
            call = ToolCall("", raw, raw)   # malformed: surfaced verbatim, the gateway decides what to do with it
        delta.tool_calls.append(call)
        self.tool_calls.append(call)

    def feed(self, text: str) -> ParsedDelta:
        delta = ParsedDelta()
        if self.stopped:
            return delta
        buf = self._hold + text
        self._hold = ""
        markers = list(self.TAGS) + (self.stop if self.mode == "content" else [])
        while buf:
            # earliest complete marker
            pos, hit = -1, None
            for m in markers:
                p = buf.find(m)
                if p >= 0 and (pos < 0 or p < pos or (p == pos and len(m) > len(hit))):
                    pos, hit = p, m
            if hit is None:
                # hold back a suffix that is a proper prefix of some marker
                keep = 0
                for m in markers:
                    for n in range(min(len(m) - 1, len(buf)), 0, -1):
                        if buf.endswith(m[:n]):
                            keep = max(keep, n)
                            break
                self._emit(delta, buf[:len(buf) - keep])
                self._hold = buf[len(buf) - keep:]
                break
            self._emit(delta, buf[:pos])
            buf = buf[pos + len(hit):]
            if hit in self.stop and self.mode == "content":
                self.stopped = True
                break
            if hit == "<think>":
                self.mode = "reasoning"
            elif hit == "</think>":
                self.mode = "content"
                buf = buf.lstrip("\n") if buf else buf
                if not buf:
                    self._strip_newlines = True
            elif hit == "<tool_call>":
                self.mode = "tool"
            elif hit == "</tool_call>":
                self._close_tool(delta)
                self.mode = "content"
            markers = list(self.TAGS) + (self.stop if self.mode == "content" else [])
        if getattr(self, "_strip_newlines", False) and delta.content:
            stripped = delta.content.lstrip("\n")
            self.content = self.content[: len(self.content) - len(delta.content)] + stripped
            delta.content = stripped
            if stripped:
                self._strip_newlines = False
        return delta

    def finish(self) -> ParsedDelta:
        """End of generation: flush held-back text (an unterminated tool frame is surfaced as content)."""
        delta = ParsedDelta()
        if self.stopped:
            return delta
        tail, self._hold = self._hold, ""
        if self.mode == "tool":
            self.mode = "content"
            tail = "<tool_call>" + self._tool + tail
            self._tool = ""
        self._emit(delta, tail)
        return delta
