"""Security stack: prompt / output filter (``ai_filter``), crypto primitives incl. the post-quantum schemes
(``crypto``), host-side services (``services``: integrity, rate limiting, firewall, vault, audit log, signed updates,
LTL checker, fuzzer), bytecode obfuscation and sealing (``obfuscation``) and the smaller services (``extras``: chaos
experiments, zero trust, audit ledger, threat intelligence, incidents, compliance, attestation)."""
from . import ai_filter, crypto, extras, obfuscation, services  # noqa: F401
