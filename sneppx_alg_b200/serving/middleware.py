"""Security middleware for the gateway (the reference's ``security_middleware.py`` / ``api_gateway.py``): one
``check`` call applies firewall rules, per-client rate limiting with temporary bans, API-key scopes and the prompt
filter, and records usage and an audit line. Optional stages from ``security.ai_extensions``: a jailbreak detector
that also looks inside base64 / hex / rot13 / URL-escaped payloads, a prompt policy, and a guard that redacts secrets
and personal data from generated text (``screen_output``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..security.ai_filter import PromptFilter
from ..security.services import ApiKeyStore, AuditLogger, DDoSMitigator, Firewall, UsageTracker


@dataclass
class Decision:
    allowed: bool
    status: int = 200
    reason: str = ""


class SecurityMiddleware:
    def __init__(self, firewall: Optional[Firewall] = None, limiter: Optional[DDoSMitigator] = None,
                 keys: Optional[ApiKeyStore] = None, audit: Optional[AuditLogger] = None, prompt_filter=None,
                 max_prompt_chars=32768, jailbreak_detector=None, prompt_policy=None, extraction_guard=None):
        self.firewall, self.limiter, self.keys, self.audit = firewall, limiter, keys, audit
        self.jailbreak, self.policy, self.guard = jailbreak_detector, prompt_policy, extraction_guard
        self.filter = prompt_filter or PromptFilter()
        self.usage = UsageTracker()
        self.max_prompt_chars = max_prompt_chars

    def check(self, client_ip: str, port: int, api_key: Optional[str], prompt: str, scope="generate") -> Decision:
        d = self._decide(client_ip, port, api_key, prompt, scope)
        if self.audit is not None:
            self.audit.log(client_ip, "request", allowed=d.allowed, status=d.status, reason=d.reason)
        return d

    def _decide(self, ip, port, key, prompt, scope):
        if self.firewall is not None and self.firewall.decide(ip, port) != "allow":
            return Decision(False, 403, "firewall")
        if self.limiter is not None and not self.limiter.check(ip):
            return Decision(False, 429, "rate limit")
        if self.keys is not None and not (key and self.keys.check(key, scope)):
            return Decision(False, 401, "api key")
        if len(prompt) > self.max_prompt_chars:
            return Decision(False, 413, "prompt too large")
        res = self.filter.check(prompt)
        if not res.allowed:
            return Decision(False, 400, "prompt filter: " + ",".join(res.reasons))
        if self.policy is not None:
            ok, why = self.policy.enforce(prompt)
            if not ok:
                return Decision(False, 400, "prompt policy: " + why)
        if self.jailbreak is not None and self.jailbreak.detect(prompt):
            return Decision(False, 400, "jailbreak pattern")
        return Decision(True)

    def screen_output(self, text: str) -> str:
        """Generated text with secrets / personal data replaced by placeholders when an extraction guard is set."""
        return text if self.guard is None else self.guard.redact(text)

    def record(self, owner: str, prompt_tokens: int, completion_tokens: int):
        self.usage.record(owner, prompt_tokens, completion_tokens)
