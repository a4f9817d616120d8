"""Host side of the stage-machine megakernel (`include/mk_stage.h`): descriptor mirror, quantisers,
tile packers and the program builder / runtime shared by the 27B, 35B-A3B and 26B-A4B engines."""
