"""S5 AI sanitiser hooks used by the serving path: prompt filter (injection / jailbreak patterns, length and
character-class limits) and output verifier (secret / PII patterns, repetition). Host-side and rule-based, like the
reference's ``PromptFilter`` / ``OutputVerifier`` (security/ai/*.c, interface_bindings/s5_safety.py), which the server
calls before and after generation (interface_bindings/inference_server.py:186-198)."""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import List

_INJECTION = [r"ignore (all|any|previous|above) (instructions|prompts)", r"disregard (the )?(system|previous) prompt",
              r"you are now (dan|developer mode)", r"reveal (your|the) (system prompt|hidden instructions)",
              r"<\s*script\b", r"\bBEGIN (RSA|OPENSSH) PRIVATE KEY\b"]
_SECRETS = [r"\bAKIA[0-9A-Z]{16}\b", r"\bsk-[A-Za-z0-9]{20,}\b", r"-----BEGIN [A-Z ]*PRIVATE KEY-----",
            r"\b\d{3}-\d{2}-\d{4}\b", r"\b(?:\d[ -]*?){13,16}\b"]


@dataclass
class FilterResult:
    allowed: bool
    reasons: List[str] = field(default_factory=list)
    sanitized: str = ""
    risk: float = 0.0


class PromptFilter:
    def __init__(self, max_chars: int = 100_000, block_threshold: float = 0.5, extra_patterns=()):
        self.max_chars, self.block_threshold = max_chars, block_threshold
        self.patterns = [re.compile(p, re.I) for p in list(_INJECTION) + list(extra_patterns)]

    def check(self, prompt: str) -> FilterResult:
        reasons, risk = [], 0.0
        if len(prompt) > self.max_chars:
            reasons.append("prompt too long")
            risk = 1.0
        ctrl = sum(1 for c in prompt if ord(c) < 9 or 13 < ord(c) < 32)
        if ctrl:
            reasons.append("control characters")
            risk = max(risk, 0.3)
        for p in self.patterns:
            if p.search(prompt):
                reasons.append(f"pattern:{p.pattern[:24]}")
                risk = max(risk, 0.8)
        clean = "".join(c for c in prompt if ord(c) >= 32 or c in "\t\n\r")[: self.max_chars]
        return FilterResult(risk < self.block_threshold, reasons, clean, risk)


class OutputVerifier:
    def __init__(self, redact: bool = True, max_repeat: int = 64):
        self.redact, self.max_repeat = redact, max_repeat
        self.patterns = [re.compile(p) for p in _SECRETS]

    def verify(self, text: str) -> FilterResult:
        reasons, out = [], text
        for p in self.patterns:
            if p.search(out):
                reasons.append(f"secret:{p.pattern[:16]}")
                if self.redact:
                    out = p.sub("[REDACTED]", out)
        m = re.search(r"(.)\1{%d,}" % self.max_repeat, out)
        if m:
            reasons.append("degenerate repetition")
        return FilterResult(not reasons or self.redact, reasons, out, 0.6 if reasons else 0.0)
