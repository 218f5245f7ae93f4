"""A vision-language model as the pairwise judge of the renderer benchmark.

The harness in ``eval.benchmark`` takes any callable; this module is the production one.  A pair is shown to the
model as still images, not as video files: every video becomes ONE contact sheet (evenly spaced frames, first and last
included, tiled left to right then top to bottom with the frame index burnt into no pixel -- the order is stated in
the prompt), so a request is four images (structure, first frame, position A, position B) and a few hundred words.

  request     an OpenAI-compatible ``chat/completions`` body; images are inline PNG data URLs; temperature 0.
  answer      the model must reply with one JSON object ``{question id: "A" | "B" | "tie"}``.  The parser takes the
              first balanced ``{...}`` of the reply, requires every asked question, and accepts nothing but the three
              values (case-insensitive); anything else is a ``JudgeAnswerError`` and the request is retried.
  transport   ``transport(url, headers, body_bytes) -> (status, body_bytes)``; the default is ``urllib``.  429 and 5xx
              are retried with doubling delays, other statuses fail at once.
  resuming    ``RecordedJudge`` appends every answer to a JSONL file keyed by (case, digest of the two renders in
              position order, questions); a rerun answers recorded pairs from the file and asks only the rest, so an
              interrupted pass costs nothing twice and a replaced render is asked again.

Reference behaviour: four questions asked in both orders, answers appended to a JSONL and skipped on rerun
(eval/solar_renderer/judge.py:30-190).
"""
from __future__ import annotations

import base64
import hashlib
import io
import json
import time
import urllib.error
import urllib.request
from pathlib import Path
from typing import Callable, Dict, Mapping, Optional, Sequence, Tuple

import numpy as np

from .benchmark import Case

QUESTIONS: Dict[str, str] = {
    "q1_visual_quality": "Which video looks better as a video: sharper, more natural, fewer artefacts and less flicker?",
    "q2_structure_motion": "Which video follows the layout and the motion of the structure video more closely?",
    "q3_first_frame": "Which video keeps the look of the given first frame (identity, colours, lighting) better over time?",
    "q4_overall": "All things considered, which video is the better render of this prompt under this structure?",
}

Transport = Callable[[str, Mapping[str, str], bytes], Tuple[int, bytes]]


class JudgeAnswerError(ValueError):
    pass


class JudgeTransportError(RuntimeError):
    def __init__(self, status: int, detail: str):
        super().__init__(f"judge endpoint answered {status}: {detail[:200]}")
        self.status = status


# ------------------------------------------------------------------------------------------------ images
def sheet_indices(frames: int, cells: int) -> Tuple[int, ...]:
    """``cells`` evenly spaced frame indices with both ends; fewer when the clip is shorter."""
    if frames < 1 or cells < 1:
        raise ValueError("a clip and a sheet both need at least one frame")
    if frames <= cells:
        return tuple(range(frames))
    if cells == 1:
        return (0,)
    return tuple(round(i * (frames - 1) / (cells - 1)) for i in range(cells))


def contact_sheet(frames: np.ndarray, cells: int = 8, columns: int = 4, cell_width: int = 320) -> np.ndarray:
    """[T, H, W, 3] uint8 -> one uint8 image of ``cells`` frames; unused cells of the last row stay black."""
    if frames.ndim != 4 or frames.shape[-1] != 3 or frames.dtype != np.uint8:
        raise ValueError("frames must be [T, H, W, 3] uint8")
    picks = sheet_indices(frames.shape[0], cells)
    h, w = frames.shape[1:3]
    ch, cw = max(1, round(h * cell_width / w)), cell_width
    ys = np.minimum((np.arange(ch) + 0.5) * h / ch, h - 1).astype(np.int64)
    xs = np.minimum((np.arange(cw) + 0.5) * w / cw, w - 1).astype(np.int64)
    columns = min(columns, len(picks))
    rows = -(-len(picks) // columns)
    sheet = np.zeros((rows * ch, columns * cw, 3), np.uint8)
    for n, t in enumerate(picks):
        r, c = divmod(n, columns)
        sheet[r * ch:(r + 1) * ch, c * cw:(c + 1) * cw] = frames[t][ys][:, xs]
    return sheet


def png_data_url(image: np.ndarray) -> str:
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray(image).save(buf, format="PNG", optimize=False)
    return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()


def _default_frames(path: str) -> np.ndarray:
    from .run_metrics import read_video
    return read_video(path)


def _default_image(path: str) -> np.ndarray:
    from PIL import Image
    return np.asarray(Image.open(path).convert("RGB"))


# ------------------------------------------------------------------------------------------------ request / answer
def build_prompt(prompt: str, questions: Sequence[str], cells: int) -> str:
    unknown = [q for q in questions if q not in QUESTIONS]
    if unknown:
        raise KeyError(f"unknown judge questions: {unknown}")
    asked = "\n".join(f"- {q}: {QUESTIONS[q]}" for q in questions)
    keys = ", ".join(f'"{q}": "A" | "B" | "tie"' for q in questions)
    return (
        "You compare two renders of one scene. Image 1 is the structure video, image 2 the given first frame, image 3 "
        f"render A, image 4 render B. Every video is shown as up to {cells} evenly spaced frames from first to last, "
        "read left to right, then top to bottom.\n"
        f"Prompt of the scene: {prompt}\n"
        f"Questions:\n{asked}\n"
        "Judge only what is visible. The position of a render (A or B) carries no information. Say tie when you cannot "
        "tell the two apart on a question.\n"
        f"Reply with one JSON object and nothing else: {{{keys}}}")


def build_request(model: str, text: str, images: Sequence[str], max_tokens: int = 200) -> dict:
    content = [{"type": "text", "text": text}] + [{"type": "image_url", "image_url": {"url": url}} for url in images]
    return {"model": model, "temperature": 0, "max_tokens": int(max_tokens), "messages": [{"role": "user", "content": content}]}


def _first_object(text: str) -> str:
    start = text.find("{")
    depth, quoted, escaped = 0, False, False
    for i in range(max(start, 0), len(text) if start >= 0 else 0):
        ch = text[i]
        if quoted:
            if escaped:
                escaped = False
            elif ch == "\\":
                escaped = True
            elif ch == '"':
                quoted = False
        elif ch == '"':
            quoted = True
        elif ch == "{":
            depth += 1
        elif ch == "}":
            depth -= 1
            if depth == 0:
                return text[start:i + 1]
    raise JudgeAnswerError("the reply holds no JSON object")


def parse_answer(text: str, questions: Sequence[str]) -> Dict[str, str]:
    try:
        doc = json.loads(_first_object(text))
    except json.JSONDecodeError as exc:
        raise JudgeAnswerError(f"the reply is not JSON: {exc}") from None
    out = {}
    for q in questions:
        value = doc.get(q)
        word = value.strip().lower() if isinstance(value, str) else None
        if word not in ("a", "b", "tie"):
            raise JudgeAnswerError(f"{q} was answered {value!r}")
        out[q] = "tie" if word == "tie" else word.upper()
    return out


def reply_text(body: bytes) -> str:
    try:
        doc = json.loads(body)
        content = doc["choices"][0]["message"]["content"]
    except (ValueError, KeyError, IndexError, TypeError):
        raise JudgeAnswerError("the endpoint's body is not a chat completion") from None
    if isinstance(content, list):                         # some servers answer in parts
        content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
    if not isinstance(content, str):
        raise JudgeAnswerError("the completion carries no text")
    return content


def urllib_transport(url: str, headers: Mapping[str, str], body: bytes, timeout: float = 300.0) -> Tuple[int, bytes]:
    req = urllib.request.Request(url, data=body, headers=dict(headers), method="POST")
    try:
        with urllib.request.urlopen(req, timeout=timeout) as resp:
            return resp.status, resp.read()
    except urllib.error.HTTPError as exc:
        return exc.code, exc.read()


class HTTPJudge:
    """``judge(case, video_a, video_b, questions) -> {question: "A" | "B" | "tie"}`` over a chat-completions endpoint."""

    def __init__(self, endpoint: str, model: str, *, api_key: Optional[str] = None, transport: Transport = urllib_transport,
                 cells: int = 8, attempts: int = 4, first_delay: float = 2.0, sleep: Callable[[float], None] = time.sleep,
                 frames_of: Callable[[str], np.ndarray] = _default_frames, image_of: Callable[[str], np.ndarray] = _default_image):
        if attempts < 1:
            raise ValueError("at least one attempt is required")
        self.url = endpoint.rstrip("/") + ("" if endpoint.rstrip("/").endswith("/chat/completions") else "/chat/completions")
        self.model, self.transport, self.cells = model, transport, int(cells)
        self.attempts, self.first_delay, self.sleep = int(attempts), float(first_delay), sleep
        self.frames_of, self.image_of = frames_of, image_of
        self.headers = {"Content-Type": "application/json", **({"Authorization": f"Bearer {api_key}"} if api_key else {})}
        self._shared: Dict[str, Tuple[str, str]] = {}     # the structure sheet and the first frame of the last case
        self.requests = 0

    def _case_images(self, case: Case) -> Tuple[str, str]:
        if case.key not in self._shared:
            self._shared = {case.key: (png_data_url(contact_sheet(self.frames_of(case.condition), self.cells)),
                                       png_data_url(self.image_of(case.first_frame)))}
        return self._shared[case.key]

    def __call__(self, case: Case, video_a: str, video_b: str, questions: Sequence[str]) -> Dict[str, str]:
        structure, first = self._case_images(case)
        sheets = [png_data_url(contact_sheet(self.frames_of(v), self.cells)) for v in (video_a, video_b)]
        body = json.dumps(build_request(self.model, build_prompt(case.prompt, questions, self.cells),
                                        [structure, first, *sheets])).encode()
        delay, problem = self.first_delay, None
        for attempt in range(self.attempts):
            if attempt:
                self.sleep(delay)
                delay *= 2
            self.requests += 1
            status, reply = self.transport(self.url, self.headers, body)
            if status == 429 or status >= 500:
                problem = JudgeTransportError(status, reply.decode("utf-8", "replace"))
                continue
            if status != 200:
                raise JudgeTransportError(status, reply.decode("utf-8", "replace"))
            try:
                return parse_answer(reply_text(reply), questions)
            except JudgeAnswerError as exc:
                problem = exc
        raise problem


# ------------------------------------------------------------------------------------------------ resuming
def _file_digest(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        for block in iter(lambda: fh.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()[:32]


class RecordedJudge:
    """Wraps a judge; answers are appended to ``log`` (JSONL) and recorded pairs are never asked again."""

    def __init__(self, judge, log, *, judge_id: str = ""):
        self.judge, self.log, self.judge_id = judge, Path(log), str(judge_id)
        self.known: Dict[str, Dict[str, str]] = {}
        self.asked = self.reused = 0
        if self.log.is_file():
            raw = self.log.read_bytes()
            if raw and not raw.endswith(b"\n"):          # an append that was cut short: drop it, that pair is asked again
                raw = raw[:raw.rfind(b"\n") + 1]
                with self.log.open("r+b") as fh:
                    fh.truncate(len(raw))
            for n, line in enumerate(raw.decode().splitlines()):
                try:
                    row = json.loads(line)
                    self.known[row["key"]] = dict(row["answer"])
                except (ValueError, KeyError, TypeError):
                    raise ValueError(f"{self.log}: line {n + 1} is damaged") from None

    def _key(self, case: Case, video_a: str, video_b: str, questions: Sequence[str]) -> str:
        doc = [self.judge_id, case.key, _file_digest(video_a), _file_digest(video_b), list(questions)]
        return hashlib.sha256(json.dumps(doc, separators=(",", ":")).encode()).hexdigest()[:32]

    def __call__(self, case: Case, video_a: str, video_b: str, questions: Sequence[str]) -> Dict[str, str]:
        key = self._key(case, video_a, video_b, questions)
        if key in self.known:
            self.reused += 1
            return dict(self.known[key])
        answer = dict(self.judge(case, video_a, video_b, questions))
        self.asked += 1
        self.log.parent.mkdir(parents=True, exist_ok=True)
        with self.log.open("a") as fh:
            fh.write(json.dumps({"key": key, "case": case.key, "a": Path(video_a).name,
                                 "b": Path(video_b).name, "answer": answer}, sort_keys=True) + "\n")
            fh.flush()
        self.known[key] = answer
        return answer


# ------------------------------------------------------------------------------------------------ command line
def main(argv=None) -> int:
    """``python -m solarwm_b200.eval.judge_client --root R --a NAME=DIR --b NAME=DIR --endpoint URL --model M --out DIR``"""
    import argparse
    import os
    from .benchmark import judge_pairs, load_cases, net_preference
    ap = argparse.ArgumentParser(prog="solar-eval-judge")
    ap.add_argument("--root", required=True)
    ap.add_argument("--a", required=True, help="method=renders directory")
    ap.add_argument("--b", required=True, help="method=renders directory")
    ap.add_argument("--endpoint", required=True)
    ap.add_argument("--model", required=True)
    ap.add_argument("--api-key-env", default="JUDGE_API_KEY")
    ap.add_argument("--split", default="all")
    ap.add_argument("--questions", default=",".join(QUESTIONS))
    ap.add_argument("--cells", type=int, default=8)
    ap.add_argument("--out", required=True)
    args = ap.parse_args(argv)
    (name_a, dir_a), (name_b, dir_b) = (spec.split("=", 1) for spec in (args.a, args.b))
    questions = [q for q in args.questions.split(",") if q]
    out = Path(args.out)
    judge = RecordedJudge(HTTPJudge(args.endpoint, args.model, api_key=os.environ.get(args.api_key_env), cells=args.cells),
                          out / f"answers-{name_a}-vs-{name_b}.jsonl", judge_id=f"{args.model}:{args.cells}")
    rows = judge_pairs(load_cases(args.root, args.split), dir_a, dir_b, judge, questions, a=name_a, b=name_b)
    report = {"a": name_a, "b": name_b, "model": args.model, "asked": judge.asked, "reused": judge.reused, "rows": rows,
              "net": {q: net_preference(rows, q, a=name_a, b=name_b) for q in questions} if rows else {}}
    (out / f"verdicts-{name_a}-vs-{name_b}.json").write_text(json.dumps(report, indent=1, sort_keys=True))
    print(json.dumps({"cases": len(rows), "asked": judge.asked, "reused": judge.reused,
                      **{q: round(v["net"], 4) for q, v in report["net"].items()}}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
