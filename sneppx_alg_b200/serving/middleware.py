"""Security middleware for the gateway (the reference's ``security_middleware.py`` / ``api_gateway.py``): one
``check`` call applies firewall rules, per-client rate limiting with temporary bans, API-key scopes and the prompt
filter, and records usage and an audit line."""
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
                 max_prompt_chars=32768):
        self.firewall, self.limiter, self.keys, self.audit = firewall, limiter, keys, audit
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
        return Decision(True)

    def record(self, owner: str, prompt_tokens: int, completion_tokens: int):
        self.usage.record(owner, prompt_tokens, completion_tokens)
