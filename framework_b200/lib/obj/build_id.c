__attribute__((visibility("default"))) const char *mni_b200_build_id(void) { return "2e9c919172fa2f00b2649c323e60c9bd71f73ec5b81431f96505819270f2f8d8"; }
