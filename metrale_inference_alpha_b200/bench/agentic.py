"""Agentic benchmark: a tool-using agent loop against a sandboxed virtual workspace.

Each task gives the model a goal, a small in-memory file system and four tools (``list_files``,
``read_file``, ``write_file``, ``finish``). The harness runs the chat loop — model turn, tool execution,
tool result appended — until the model calls ``finish``, stops calling tools, or the turn budget runs out,
then scores the final workspace with the task's checker. Nothing touches the real file system or a shell:
tools are pure functions on the task's dict, paths are normalised and may not leave the workspace root.

A trace (every model message, every tool call with its result or error, token usage and wall time per
turn) is returned with the score so a failed run can be read turn by turn; truncated tool results and
repeated identical calls are counted as diagnostics. ``ask`` is any callable ``(messages, tools) ->
assistant message`` (see ``function_calling.app_asker`` / ``http_asker``).

Reference: ``crates/bench/src/benchmarks/agentic/{agent,agent_tools,agent_shell,score,trace,verdict}.rs``.
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from .function_calling import Asker, calls_of_message

MAX_RESULT_CHARS = 4000

TOOLS = [
    {"type": "function", "function": {"name": "list_files", "description": "List the files of the workspace.",
                                      "parameters": {"type": "object", "properties": {}, "required": []}}},
    {"type": "function", "function": {"name": "read_file", "description": "Read a file of the workspace.",
                                      "parameters": {"type": "object", "properties": {"path": {"type": "string"}}, "required": ["path"]}}},
    {"type": "function", "function": {"name": "write_file", "description": "Create or replace a file of the workspace.",
                                      "parameters": {"type": "object", "properties": {"path": {"type": "string"}, "content": {"type": "string"}},
                                                     "required": ["path", "content"]}}},
    {"type": "function", "function": {"name": "finish", "description": "Declare the task done.",
                                      "parameters": {"type": "object", "properties": {"summary": {"type": "string"}}, "required": []}}},
]


@dataclass
class Task:
    id: str
    goal: str
    files: Dict[str, str]
    check: Callable[[Dict[str, str]], bool]
    max_turns: int = 8


@dataclass
class Trace:
    task: str
    turns: List[dict] = field(default_factory=list)
    finished: bool = False
    reason: str = ""
    passed: bool = False
    repeated_calls: int = 0
    truncated_results: int = 0
    tool_errors: int = 0
    seconds: float = 0.0


def norm_path(path: str) -> str:
    """Workspace-relative normal form; raises on a path that leaves the root."""
    if not isinstance(path, str) or not path.strip():
        raise ValueError("empty path")
    stack: List[str] = []
    for part in path.strip().replace("\\", "/").split("/"):
        if part in ("", "."):
            continue
        if part == "..":
            if not stack:
                raise ValueError(f"path {path!r} is outside the workspace")
            stack.pop()
        else:
            stack.append(part)
    if not stack:
        raise ValueError(f"path {path!r} names no file")
    p = "/".join(stack)
    return p


def run_tool(files: Dict[str, str], name: str, args: dict) -> str:
    if name == "list_files":
        return "\n".join(sorted(files)) or "(empty)"
    if name == "read_file":
        p = norm_path(args.get("path"))
        if p not in files:
            raise FileNotFoundError(f"no such file: {p}")
        return files[p]
    if name == "write_file":
        p = norm_path(args.get("path"))
        content = args.get("content")
        if not isinstance(content, str):
            raise ValueError("content must be a string")
        files[p] = content
        return f"wrote {len(content)} characters to {p}"
    if name == "finish":
        return "ok"
    raise ValueError(f"unknown tool {name!r}")


def run_task(task: Task, ask: Asker, system: str = "You are an agent working in a small workspace. Use the tools; call finish when done.") -> Trace:
    files = dict(task.files)
    msgs: List[dict] = [{"role": "system", "content": system}, {"role": "user", "content": task.goal}]
    tr = Trace(task.id)
    seen = set()
    t0 = time.perf_counter()
    for turn in range(task.max_turns):
        t1 = time.perf_counter()
        try:
            msg = ask(msgs, TOOLS)
        except Exception as e:
            tr.reason = f"request failed: {e}"
            break
        calls = calls_of_message(msg)
        rec = {"turn": turn, "content": msg.get("content"), "calls": [], "seconds": time.perf_counter() - t1}
        tr.turns.append(rec)
        msgs.append({"role": "assistant", "content": msg.get("content") or "", "tool_calls": msg.get("tool_calls") or []})
        if not calls:
            tr.reason = "the model stopped calling tools"
            break
        for i, c in enumerate(calls):
            args = c.get("arguments")
            try:
                args = json.loads(args) if isinstance(args, str) else (args or {})
                key = (c["name"], json.dumps(args, sort_keys=True))
                if key in seen and c["name"] != "finish":
                    tr.repeated_calls += 1
                seen.add(key)
                res, err = run_tool(files, c["name"], args), False
            except Exception as e:
                res, err = f"error: {e}", True
                tr.tool_errors += 1
            if len(res) > MAX_RESULT_CHARS:
                res = res[:MAX_RESULT_CHARS] + "\n[truncated]"
                tr.truncated_results += 1
            rec["calls"].append({"name": c.get("name"), "arguments": args, "result": res, "error": err})
            tc_id = ((msg.get("tool_calls") or [{}] * (i + 1))[i] or {}).get("id") or f"call_{turn}_{i}"
            msgs.append({"role": "tool", "tool_call_id": tc_id, "content": res})
            if c.get("name") == "finish" and not err:
                tr.finished = True
        if tr.finished:
            tr.reason = "finish"
            break
    else:
        tr.reason = "turn budget exhausted"
    tr.seconds = time.perf_counter() - t0
    try:
        tr.passed = bool(task.check(files))
    except Exception:
        tr.passed = False
    return tr


def builtin_tasks() -> List[Task]:
    return [
        Task("rename_constant", "In config.py, change TIMEOUT from 30 to 60. Leave everything else as it is.",
             {"config.py": "NAME = 'svc'\nTIMEOUT = 30\nRETRIES = 3\n"},
             lambda f: "TIMEOUT = 60" in f.get("config.py", "") and "RETRIES = 3" in f.get("config.py", "")),
        Task("create_readme", "Create README.md that mentions the project name found in setup.cfg.",
             {"setup.cfg": "[metadata]\nname = orbital\nversion = 1.2\n"},
             lambda f: "orbital" in f.get("README.md", "").lower()),
        Task("sum_numbers", "numbers.txt holds one integer per line. Write their sum to total.txt.",
             {"numbers.txt": "4\n8\n15\n16\n23\n42\n"},
             lambda f: f.get("total.txt", "").strip() == "108"),
    ]


def score(traces: Sequence[Trace]) -> dict:
    n = len(traces)
    return {"n": n, "passed": sum(t.passed for t in traces), "pass_rate": (sum(t.passed for t in traces) / n) if n else 0.0,
            "finished": sum(t.finished for t in traces), "mean_turns": (sum(len(t.turns) for t in traces) / n) if n else 0.0,
            "tool_errors": sum(t.tool_errors for t in traces), "repeated_calls": sum(t.repeated_calls for t in traces),
            "truncated_results": sum(t.truncated_results for t in traces),
            "tasks": {t.task: {"passed": t.passed, "turns": len(t.turns), "reason": t.reason} for t in traces}}


def run_suite(ask: Asker, tasks: Optional[Sequence[Task]] = None) -> dict:
    traces = [run_task(t, ask) for t in (tasks or builtin_tasks())]
    out = score(traces)
    out["traces"] = traces
    return out
