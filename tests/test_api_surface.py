"""The public names of every façade namespace (the surface a user of the reference library relies on)."""
import importlib
import inspect

import pytest

SURFACE = {
    "serialization": "state_dict from_state_dict register_serializer register_template_restored lookup_serializer resolve_serializer",
    "types": "ClipState ClippedPytree MaxNorm NoiseState NoiseStddev NoisedPytree ParamPath PerGroup SecondMomentClippingOutput "
             "SecondMomentNoiseOutput TensorPytree clipped noised",
    "pytree": "ParamPath global_norm merge param_path param_path_display partition tree_flatten tree_flatten_with_paths tree_leaves "
              "tree_map tree_map_with_path tree_structure tree_unflatten",
    "random": "key fold_in split generator_from_key random_key set_reproducible_pytorch_seed",
    "functional": "make_functional with_batch_dim empty_collate",
    "distributed": "all_reduce barrier gather_for_metrics get_rank get_world_size is_distributed is_main_process local_shard "
                   "num_processes process_index reduce_pytree reduce_pytree_ sum_gradients sum_gradients_ sync wait_for_everyone "
                   "reduce_scalar all_reduce_ gather_tensors gather_pytree assert_pytree_equal assert_scalar_equal sync_object",
    "profiling": "PerfStage PerfState PerfTracker StepPerf empty_cache get_memory_stats perf_tracker print_memory reset_peak_memory step_perf",
    "precision": "LossScaler LossScalerState all_finite loss_scaler",
    "scheduling": "constant_schedule cosine_schedule exponential_schedule inverse_sqrt_schedule linear_schedule one_minus_sqrt_schedule "
                  "polynomial_schedule warmup_stable_decay with_restarts with_warmup",
    "device": "DeviceCapabilities device_capabilities fused_kernels_available sdpa_autocast_under_vmap_broken",
    "accounting": "amplification calibration composition discretization mechanisms Accountant set_discretization get_discretization "
                  "eps_delta identity nonprivate repeat compose cached per_step epsilon_budget delta_budget advantage_budget beta_budget "
                  "risk_budget register_budget_serializer calibrate",
    "dpsgd": "accounting clipping noise sampling adaptive_clipped_grad auto_clipped_grad clipped_grad per_group gaussian_noise PoissonSampler",
    "dpsgd.accounting": "adaclip gaussian k_out_of_t parallel_poisson poisson random_allocation",
    "dpsgd.sampling": "KOutOfTSampler PoissonSampler RandomAllocationSampler",
    "dpftrl": "accounting clipping noise sampling clipped_grad auto_clipped_grad per_group mf_gaussian_noise band_mf_strategy bisr_strategy "
              "bsr_strategy blt_strategy identity_strategy lambda_cgd_strategy BallsInBinsSampler BMinSepSampler CyclicPoissonSampler "
              "SequentialBatchSampler",
    "dpftrl.accounting": "b_min_sep balls_in_bins mf_gaussian per_step poisson",
    "optimizers": "adadelta adafactor adagrad adam adamw ademamix lion radam rmsprop schedule_free sgd types make_optimizer_chain apply_updates",
    "patches": "apply_model_patches apply_peft_model_patches apply_runtime_patches apply_transformers_model_patches is_runtime_patched",
    "patches.kernels": "ACTIVATION_SWIGLU ACTIVATION_GEGLU_EXACT ACTIVATION_GEGLU_APPROX opaque_cross_entropy_loss opaque_fused_add_rms_norm "
                       "opaque_geglu_approx opaque_geglu_exact opaque_linear_cross_entropy_loss opaque_lora_mlp opaque_lora_qkv opaque_lora_w "
                       "opaque_moe opaque_rms_norm opaque_rope opaque_rope_qk opaque_slow_rope opaque_swiglu opaque_selective_log_softmax",
    "transformers": "DPTrainer TrainingArguments trl",
    "transformers.trl": "SFTTrainer SFTConfig DPOTrainer DPOConfig",
    "alignment": "data dpo metric sft",
    "auditing": "canary_scores coin_flip gradient_scores loss_scores one_run",
}


@pytest.mark.parametrize("namespace", sorted(SURFACE))
def test_namespace_exports(namespace):
    mod = importlib.import_module(f"opaque_b200.{namespace}")
    missing = [n for n in SURFACE[namespace].split() if not hasattr(mod, n)]
    assert not missing, f"opaque_b200.{namespace} lacks {missing}"


def test_key_signatures():
    from opaque_b200 import accounting, dpftrl, dpsgd, functional, optimizers
    from opaque_b200.transformers import DPTrainer

    def params(fn):
        return list(inspect.signature(fn).parameters)
    assert params(dpsgd.clipped_grad)[:3] == ["loss_fn", "argnums", "has_aux"]
    for name in ("clipping_norm", "normalize_by", "batch_argnums", "return_aux", "return_stats", "second_moment", "pre_clipping_transform",
                 "microbatch_size", "dtype", "compute_dtype"):
        assert name in params(dpsgd.clipped_grad), name
    for name in ("R", "gamma", "normalize_by", "batch_argnums", "microbatch_size"):
        assert name in params(dpsgd.auto_clipped_grad), name
    for name in ("initial_clipping_norm", "target_quantile", "learning_rate", "clipping_norm_min", "clipping_norm_max", "fraction_noise_std", "key"):
        assert name in params(dpsgd.adaptive_clipped_grad), name
    assert set(params(dpsgd.gaussian_noise)) >= {"noise_multiplier", "key", "bound", "compute_dtype"}
    assert set(params(dpftrl.mf_gaussian_noise)) >= {"grad_template", "strategy", "n_steps", "min_sep", "max_participations", "noise_multiplier",
                                                     "key", "compute_dtype", "second_moment_strategy"}
    assert params(accounting.calibrate) == ["budget", "process", "param_min", "param_max", "tolerance", "max_iterations", "prefix"]
    assert params(functional.make_functional) == ["mod", "disable_autograd_tracking", "partition_trainable"]
    assert set(params(optimizers.adamw)) >= {"lr", "betas", "eps", "weight_decay", "decoupled_weight_decay", "update_rms_clip", "noise_bias_correction"}
    assert params(DPTrainer.__init__)[1:] == ["model", "args", "data_collator", "train_dataset", "eval_dataset", "processing_class",
                                              "compute_loss_func", "compute_metrics", "callbacks", "optimizers", "optimizer_cls_and_kwargs",
                                              "preprocess_logits_for_metrics"]
    for m in ("train", "evaluate", "predict", "save_model", "training_step"):
        assert callable(getattr(DPTrainer, m))


def test_native_accounting_stub_declares_every_public_name():
    """``accounting/_native.pyi`` is the typed surface of the C++ core: nothing public is missing from it."""
    import ast
    import pathlib

    from opaque_b200.accounting import _native
    stub = pathlib.Path(_native.__file__).with_name("_native.pyi")
    tree = ast.parse(stub.read_text())
    declared = {n.name for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef))}
    public = {n for n in dir(_native) if not n.startswith("_")}
    assert public <= declared, sorted(public - declared)


SUBPATHS = {
    "alignment.dpo.collator": "preference_collator",
    "alignment.dpo.data": "extract_prompt",
    "alignment.dpo.loss": "sequence_logp fused_sequence_logp sigmoid_loss hinge_loss robust_loss ipo_loss discopop_loss chosen_nll_loss "
                          "apo_zero_loss apo_down_loss exo_loss nca_loss bco_loss sppo_loss simpo_loss odds_ratio_loss f_divergence_remap "
                          "f_divergence_logits mpo_combine wpo_weights ld_dpo_split",
    "alignment.dpo.metric": "reward_metrics",
    "alignment.dpo.reference": "compute_ref_logprobs_for_dataset ema_update_reference null_ref_context with_disabled_adapter",
    "alignment.metric": "entropy_from_logits mean_token_accuracy",
    "alignment.sft.collator": "language_modeling_collator",
    "alignment.sft.loss": "dft_loss fused_dft_loss fused_nll_loss nll_loss",
    "auditing.attacks": "gradient_scores loss_scores",
    "auditing.one_run": "one_run",
    "dpftrl.accounting.amplification": "b_min_sep balls_in_bins poisson",
    "dpftrl.accounting.mechanisms": "mf_gaussian",
    "dpftrl.clipping": "auto_clipped_grad clipped_grad per_group",
    "dpsgd.accounting.amplification": "k_out_of_t parallel_poisson poisson random_allocation",
    "dpsgd.accounting.mechanisms": "adaclip gaussian",
    "patches.peft": "apply_peft_model_patches",
    "patches.torch": "apply_checkpoint_patch is_checkpoint_patched",
    "patches.transformers": "FamilyPatchFn ForwardFactory ForwardFn ModelPatchFn ModulePatcher apply_transformers_model_patches family_name "
                            "make_apply_family_patches make_apply_model_patches register_activation_kind register_family "
                            "register_fused_add_rms_kind register_rms_norm_kind supported_families",
    "patches.transformers.runtime": "apply_collator_patches apply_grouped_mm_patches apply_masking_patches",
    "transformers.trainer.types": "EvaluationResult TrainOutput",
    "accounting.types": "Accountant AdvantageBudget BetaBudget Budget CachedProcess CalibrateResult Composed DeltaBudget DiscretizationConfig "
                        "DpHorizonProcess DpProcess EpsDelta EpsilonBudget Identity NonPrivate PerStep Repeated RiskBudget",
    "alignment.dpo.collator.types": "PreferenceBatch PreferenceExample",
    "alignment.sft.collator.types": "LMBatch LMExample",
    "auditing.types": "CanaryScores CoinFlip OneRunEstimate",
    "distributed.collectives": "all_reduce all_reduce_ barrier get_rank get_world_size is_distributed",
    "distributed.gradients": "reduce_pytree reduce_pytree_ sum_gradients sum_gradients_",
    "dpftrl.accounting.amplification.types": "BMinSep BallsInBins CyclicPoisson",
    "dpftrl.accounting.mechanisms.types": "MfGaussian",
    "dpftrl.accounting.types": "BMinSep BallsInBins CyclicPoisson MfGaussian",
    "dpftrl.clipping.fun": "auto_clipped_fun auto_scale_pytree clip_pytree clipped_fun",
    "dpftrl.clipping.types": "AutoClipState AutoClippedFunAux AutoClippedGradAux ClipPytreeAux ClippedFunAux ClippedGradAux ClippedGradFn "
                             "ClippedGradResult FixedClipState",
    "dpftrl.noise.types": "BandMfStrategy BisrStrategy BltStrategy BsrStrategy IdentityStrategy LambdaCgdStrategy MFNoiseState MfStrategy "
                          "SecondMomentMFNoiseState",
    "dpftrl.sampling.types": "PartitionType",
    "dpsgd.accounting.amplification.types": "KOutOfT ParallelPoisson Poisson RandomAllocation",
    "dpsgd.accounting.mechanisms.types": "AdaClip Gaussian",
    "dpsgd.accounting.types": "AdaClip Gaussian KOutOfT ParallelPoisson Poisson RandomAllocation",
    "dpsgd.clipping.fun": "auto_clipped_fun auto_scale_pytree clip_pytree clipped_fun",
    "dpsgd.clipping.types": "AdaptiveClipState AdaptiveClippedGradAux AutoClipState AutoClippedFunAux AutoClippedGradAux ClippingStats "
                            "ClippedGradFn ClippedGradResult FixedClipState",
    "dpsgd.noise.types": "GaussianNoiseFn GaussianNoiseInput GaussianNoiseOutput GaussianNoiseState",
    "optimizers.types": "AdEMAMixState AdadeltaState AdafactorState AdagradState AdamState LionState RAdamState RMSpropState ScheduleFreeState",
    "patches.transformers.types": "FamilyPatchFn ForwardFactory ForwardFn ModelPatchFn ModulePatcher",
    "profiling.types": "MemoryStats PerfStage PerfState PerfTracker StepPerf",
    "random.types": "RngKey",
    "scheduling.types": "ConstantSchedule CosineSchedule ExponentialSchedule InverseSqrtSchedule LinearSchedule OneMinusSqrtSchedule "
                        "PolynomialSchedule Schedule WarmupStableDecay WithRestarts WithWarmup",
}


@pytest.mark.parametrize("path", sorted(SUBPATHS))
def test_deeper_import_paths_of_the_reference_resolve(path):
    """``from opaque.<path> import name`` of the reference works as ``from opaque_b200.<path> import name``."""
    mod = importlib.import_module(f"opaque_b200.{path}")
    missing = [n for n in SUBPATHS[path].split() if not hasattr(mod, n)]
    assert not missing, f"opaque_b200.{path} lacks {missing}"


def test_facades_carry_a_version_and_one_run_stays_callable():
    import torch
    import opaque_b200
    for name in ("accounting", "alignment", "auditing", "dpftrl", "dpsgd", "transformers", "patches"):
        assert importlib.import_module(f"opaque_b200.{name}").__version__ == opaque_b200.__version__
    from opaque_b200 import auditing, patches
    from opaque_b200.auditing.one_run import one_run
    flips = auditing.coin_flip(range(40), num_canaries=20, key=__import__("opaque_b200.random", fromlist=["key"]).key(1))
    scores = auditing.canary_scores(torch.arange(20.0))
    assert auditing.one_run(scores, coin_flip=flips).num_canaries == one_run(scores, coin_flip=flips).num_canaries == 20
    assert patches.torch is torch or not hasattr(patches, "torch")        # the library's name is not shadowed
