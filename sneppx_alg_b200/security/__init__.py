"""Security stack: prompt / output filter (``ai_filter``), crypto primitives incl. the post-quantum schemes
(``crypto``), host-side services (``services``: integrity, rate limiting, firewall, vault, audit log, signed updates,
LTL checker, fuzzer), bytecode obfuscation and sealing (``obfuscation``) and the smaller services (``extras``: chaos
experiments, zero trust, audit ledger, threat intelligence, incidents, compliance, attestation). Imported on demand:
``memory`` (S1), ``monitoring`` / ``integrity_ext`` (S3), ``network`` / ``network_ext`` / ``tls13`` (S4), ``ai_safety`` / ``ai_extensions`` /
``model_watermark`` (S5), ``vault_ext`` (S6), ``updates_ext`` (S7), ``formal`` / ``formal_ext`` (S8), ``pentest`` (S9)."""
from . import ai_filter, crypto, extras, obfuscation, services  # noqa: F401
