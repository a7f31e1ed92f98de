"""The launch model of the FP8 product (host arithmetic of the C library, no GPU): which tile kernel and width a
launch takes.  The expectations are what timing both kernels on a B200 found fastest for the shapes one rank of a
FLUX-shape model sees at 1, 2, 4 and 8 GPUs (4096 image + 512 text tokens split over the ranks)."""
import pytest

from cache_dit_b200 import _native as nat

SINGLE, PAIR, FEW_ROWS = 1, 2, 3


def rank_shapes(world):
  img, txt, joint = 4096 // world, 512 // world, 4608 // world
  return {
    "dbl_qkv": [(img, 9216, 3072), (txt, 9216, 3072)],
    "dbl_out": [(img, 3072, 3072), (txt, 3072, 3072)],
    "dbl_mlp_in": [(img, 12288, 3072), (txt, 12288, 3072)],
    "dbl_mlp_out": [(img, 3072, 12288), (txt, 3072, 12288)],
    "sgl_qkv_mlp": [(joint, 21504, 3072)],
    "sgl_out": [(joint, 3072, 15360)],
  }


@pytest.fixture(autouse=True)
def _knobs_off():
  lib = nat.lib()
  lib.cdb_tuning_set_gemm_kernel(0)
  lib.cdb_tuning_set_gemm_tile_cols(0)
  yield
  lib.cdb_tuning_set_gemm_kernel(0)
  lib.cdb_tuning_set_gemm_tile_cols(0)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_rank_shard_products_take_the_kernel_that_measured_fastest(world):
  # the two launches where 256-row pair tiles need a fourth wave and 128-row tiles only three
  single_wins = {(4, "dbl_mlp_in"), (8, "sgl_qkv_mlp")}
  for name, shapes in rank_shapes(world).items():
    kind, cols = nat.fp8_gemm_plan(shapes)
    if (world, name) in single_wins:
      assert kind == SINGLE and cols == 256, (world, name, kind, cols)
    else:
      assert kind == PAIR and cols == 256, (world, name, kind, cols)


def test_few_rows_and_order_of_the_problems():
  assert nat.fp8_gemm_plan([(1, 18432, 3072)]) == (FEW_ROWS, 0)
  assert nat.fp8_gemm_plan([(4, 3072, 3072)]) == (FEW_ROWS, 0)
  assert nat.fp8_gemm_plan([(5, 3072, 3072)])[0] in (SINGLE, PAIR)
  assert nat.fp8_gemm_plan([(0, 3072, 3072)]) == (0, 0)
  a = nat.fp8_gemm_plan([(64, 12288, 3072), (512, 12288, 3072)])
  assert a == nat.fp8_gemm_plan([(512, 12288, 3072), (64, 12288, 3072)])


def test_knobs_decide_when_set():
  lib = nat.lib()
  shapes = [(576, 21504, 3072)]
  lib.cdb_tuning_set_gemm_kernel(2)
  assert nat.fp8_gemm_plan(shapes) == (PAIR, 256)
  lib.cdb_tuning_set_gemm_tile_cols(128)
  assert nat.fp8_gemm_plan(shapes) == (PAIR, 128)
  lib.cdb_tuning_set_gemm_tile_cols(80)  # a pair tile needs a multiple of 32
  with pytest.raises(Exception):
    nat.fp8_gemm_plan(shapes)
  lib.cdb_tuning_set_gemm_kernel(1)
  assert nat.fp8_gemm_plan(shapes) == (SINGLE, 80)
  lib.cdb_tuning_set_gemm_kernel(0)
  assert nat.fp8_gemm_plan(shapes) == (SINGLE, 80)  # a forced width alone means the single-CTA kernel
  assert nat.fp8_gemm_plan([(4608, 12288, 3072)])[0] == PAIR  # except for tall problems
  with pytest.raises(Exception):
    nat.fp8_gemm_plan([(576, 0, 3072)])


def test_a_narrow_product_on_few_rows_takes_a_narrower_single_cta_tile():
  # 576 x 3072 x 3072 alone: 60 full-width tiles for 148 SMs; pairs (36 tiles) win the near-tie by design
  kind, cols = nat.fp8_gemm_plan([(576, 3072, 3072)])
  assert (kind, cols) == (PAIR, 256)
  # with the pair kernel excluded the model narrows the tile until one wave is full
  nat.lib().cdb_tuning_set_gemm_kernel(1)
  kind, cols = nat.fp8_gemm_plan([(576, 3072, 3072)])
  assert kind == SINGLE and 96 <= cols <= 128 and cols % 16 == 0
