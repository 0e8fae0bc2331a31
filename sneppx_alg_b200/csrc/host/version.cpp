// Host runtime library: version / build information.
extern "C" const char* sx_host_version() { return "sneppx-host 0.1.0"; }
