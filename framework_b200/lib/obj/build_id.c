__attribute__((visibility("default"))) const char *mni_b200_build_id(void) { return "fa64b4c1b6e8a3e782d74736e3a98263b3216e0a0397f30532bf00d3189130cd"; }
