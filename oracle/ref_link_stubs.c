/*
 * TEST INFRASTRUCTURE ONLY.  Link-time stand-ins for reference symbols that live in
 * translation units outside the KV path and are therefore not compiled into
 * oracle/_ref/libwarp34_ref.so.  None of them is reachable from the KV-cache write or the
 * paged-attention entry points; they only satisfy the dynamic loader.
 *
 *   warp34_vision_fa2_prepare  defined in the reference's op_vision_fa2.cu (ViT attention),
 *                              referenced by its runtime-create routine in op_init.cu:316-322.
 */
int warp34_vision_fa2_prepare(void) { return 0; }
