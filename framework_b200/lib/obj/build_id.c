__attribute__((visibility("default"))) const char *mni_b200_build_id(void) { return "29d421111da130e27cca23639209781e1e095b066441c9ff9c1802a2c09eee0b"; }
