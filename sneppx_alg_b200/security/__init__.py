"""Security stack: prompt / output filter (``ai_filter``), crypto primitives (``crypto``), host-side services
(``services``: integrity, rate limiting, firewall, vault, audit log, signed updates, LTL checker, fuzzer)."""
from . import ai_filter, crypto, services  # noqa: F401
