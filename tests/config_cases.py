"""Inputs for the configuration loaders, shared by the fixture generator and the test."""

CACHE_CASES = {
    "nested_taylor": dict(input={"cache_config": {"Fn_compute_blocks": 1, "Bn_compute_blocks": 2, "max_warmup_steps": 4,
                                                  "warmup_interval": 2, "max_continuous_cached_steps": 2,
                                                  "residual_diff_threshold": 0.12, "enable_taylorseer": True,
                                                  "taylorseer_order": 2}}),
    "nested_mask_policy": dict(input={"cache_config": {"steps_computation_mask": "fast", "num_inference_steps": 28,
                                                       "steps_computation_policy": "static"}}),
    "nested_mask_list": dict(input={"cache_config": {"steps_computation_mask": [1, 1, 0, 0, 1, 0], "num_inference_steps": 6}}),
    "flat_legacy": dict(input={"Fn_compute_blocks": 4, "max_cached_steps": 12, "enable_taylorseer": True,
                               "enable_encoder_taylorseer": True, "taylorseer_cache_type": "hidden_states"}),
    "flat_reset": dict(input={"num_inference_steps": 30}, kwargs={"reset": True}),
    "flat_reset_taylor": dict(input={"num_inference_steps": 16, "enable_taylorseer": True, "taylorseer_order": 3,
                                     "verbose": True}, kwargs={"reset": True}),
    "unknown_keys_ignored": dict(input={"cache_config": {"Fn_compute_blocks": 2, "not_a_field": 7,
                                                         "residual_diff_threshold": None}}),
    "explicit_dbcache": dict(input={"cache_config": {"cache_type": "DBCache", "max_warmup_steps": 2}}),
    "other_sections_only": dict(input={"parallelism_config": {"ulysses_size": 1}, "attention_backend": "native"}),
    "bad_cache_type": dict(input={"cache_config": {"cache_type": "Nope"}}),
    "two_calibrators": dict(input={"cache_config": {"enable_taylorseer": True, "enable_dmd": True}}),
    "mask_policy_without_steps": dict(input={"cache_config": {"steps_computation_mask": "slow"}}),
    "empty_flat": dict(input={}),
    "not_a_config": dict(input=12),
}

PARALLEL_CASES = {
    "absent": dict(input={"cache_config": {}}),
    "check_only": dict(input={"parallelism_config": {"ulysses_size": 1}}, kwargs={"check_only": True}),
    "alias": dict(input={"parallelism_config": {"ulysses": 1, "ulysses_anything": True}}),
    "alias_conflict": dict(input={"parallelism_config": {"ulysses": 2, "ulysses_size": 4}}),
    "auto_without_group": dict(input={"parallelism_config": {"ulysses_size": "auto"}}),
    "two_autos": dict(input={"parallelism_config": {"ulysses_size": "auto", "ring_size": "auto"}}),
    "bad_size": dict(input={"parallelism_config": {"ulysses_size": "many"}}),
    "backend_name": dict(input={"parallelism_config": {"backend": "native_diffuser", "ulysses_size": 1}}),
    "bad_backend": dict(input={"parallelism_config": {"backend": "mpi"}}),
}

PARALLEL_FIELDS = ("ulysses_size", "ring_size", "tp_size", "ulysses_anything", "ulysses_float8", "ulysses_async",
                   "attention_backend")


def describe_cache(result):
  """JSON form of what `load_cache_config` returned."""
  cache, calibrator = result

  def fields(obj):
    import dataclasses
    out = {}
    for f in dataclasses.fields(obj):
      v = getattr(obj, f.name)
      if f.name == "cache_type":
        continue  # the reference leaves the name string here, this package keeps the enum
      out[f.name] = v if isinstance(v, (int, float, str, bool, list, type(None))) else str(v)
    return out

  return dict(cache=None if cache is None else fields(cache),
              calibrator=None if calibrator is None else dict(kind=type(calibrator).__name__, **fields(calibrator)))


def describe_parallel(result):
  if result is None or isinstance(result, bool):
    return result
  return dict(backend=str(result.backend), **{k: getattr(result, k) for k in PARALLEL_FIELDS})


def run_cases(module):
  """{case: description or {"error": exception class}} for both tables, using `module`'s loaders."""
  out = {"cache": {}, "parallel": {}}
  for table, cases, loader, describe in (("cache", CACHE_CASES, module.load_cache_config, describe_cache),
                                         ("parallel", PARALLEL_CASES, module.load_parallelism_config, describe_parallel)):
    for name, case in cases.items():
      try:
        out[table][name] = describe(loader(case["input"], **case.get("kwargs", {})))
      except Exception as e:  # the class of the error is part of the behaviour
        out[table][name] = {"error": type(e).__name__}
  return out
