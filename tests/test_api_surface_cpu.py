"""The public names of the reference (constructors, builder methods, presets) exist here under the
same names, so user code written against the Rust crates maps one to one."""
from axonml_b200 import autograd, data, jit, llm, nn, optim, parallel


def _missing(obj, names):
    return [f"{getattr(obj, '__name__', obj)}.{n}" for n in names.split() if not hasattr(obj, n)]


def test_nn_surface():
    m = []
    m += _missing(nn.Linear, "new with_bias from_weights")
    for c in (nn.Conv1d, nn.Conv2d, nn.MaxPool1d, nn.MaxPool2d, nn.AvgPool1d, nn.AvgPool2d, nn.BatchNorm1d, nn.BatchNorm2d,
              nn.GroupNorm, nn.RNN, nn.LSTM, nn.GRU):
        m += _missing(c, "new with_options")
    m += _missing(nn.AdaptiveAvgPool2d, "new square")
    m += _missing(nn.LayerNorm, "new single with_eps")
    m += _missing(nn.InstanceNorm2d, "new with_affine with_options")
    m += _missing(nn.Dropout, "new default_p")
    m += _missing(nn.Embedding, "new with_options from_pretrained")
    for c in (nn.RNNCell, nn.LSTMCell, nn.GRUCell):
        m += _missing(c, "new")
    m += _missing(nn.GRU, "forward_mean forward_last")
    m += _missing(nn.MultiHeadAttention, "new with_options attention")
    m += _missing(nn.LeakyReLU, "new with_slope") + _missing(nn.ELU, "new with_alpha")
    m += _missing(nn.Softmax, "new") + _missing(nn.LogSoftmax, "new")
    for c in (nn.MSELoss, nn.L1Loss, nn.CrossEntropyLoss, nn.NLLLoss, nn.BCELoss, nn.BCEWithLogitsLoss, nn.SmoothL1Loss):
        m += _missing(c, "new with_reduction compute")
    m += _missing(nn.SmoothL1Loss, "with_beta")
    m += _missing(nn.Sequential, "new add add_named push push_named iter")
    m += _missing(nn.ModuleList, "new from_vec push get iter")
    m += _missing(nn.Module, "forward parameters named_parameters num_parameters train eval set_training is_training zero_grad name")
    m += _missing(nn.Parameter, "new named from_variable name set_name variable data shape numel requires_grad grad zero_grad "
                                "update_data apply_update")
    m += _missing(nn.F, "relu leaky_relu sigmoid tanh gelu silu elu softmax log_softmax linear layer_norm dropout mse_loss "
                        "cross_entropy binary_cross_entropy adaptive_avg_pool2d")
    m += _missing(nn.init, "zeros ones constant uniform uniform_range randn normal xavier_uniform xavier_normal glorot_uniform "
                           "glorot_normal kaiming_uniform kaiming_normal he_uniform he_normal orthogonal sparse eye diag InitMode")
    assert not m, m


def test_optim_surface():
    m = []
    m += _missing(optim.SGD, "new with_momentum with_options momentum weight_decay nesterov dampening")
    m += _missing(optim.Adam, "new with_betas with_options betas eps weight_decay amsgrad")
    m += _missing(optim.AdamW, "new with_betas with_options")
    m += _missing(optim.RMSprop, "new with_alpha with_options alpha eps weight_decay momentum centered")
    m += _missing(optim.LAMB, "new with_betas with_options betas eps weight_decay bias_correction")
    m += _missing(optim.GradScaler, "new with_scale with_options growth_factor backoff_factor growth_interval enabled get_scale "
                                    "set_scale is_enabled set_enabled scale_loss unscale_grads check_grads found_inf set_found_inf "
                                    "update state_dict load_state_dict scale step")
    m += _missing(optim, "StepLR MultiStepLR ExponentialLR CosineAnnealingLR ReduceLROnPlateau OneCycleLR WarmupLR clip_grad_norm "
                         "clip_grad_value")
    assert not m, m


def test_distributed_llm_data_jit_surface():
    m = []
    m += _missing(parallel, "World ProcessGroup DistributedDataParallel GradientBucket GradientSynchronizer FullyShardedDataParallel "
                            "ColumnParallelLinear RowParallelLinear Pipeline DDP FSDP ShardingStrategy CPUOffload DeviceMesh")
    m += _missing(parallel.World, "init mock") + _missing(parallel.ProcessGroup, "with_ranks mock")
    m += _missing(parallel.DistributedDataParallel, "broadcast_buffers gradient_as_bucket_view sync_parameters sync_gradients module")
    m += _missing(parallel.FullyShardedDataParallel, "sharding_strategy cpu_offload mixed_precision gather_parameters "
                                                     "reshard_parameters sync_gradients clip_grad_norm memory_estimate")
    m += _missing(parallel.Pipeline, "from_modules schedule num_microbatches")
    m += _missing(llm, "LLaMAConfig GPT2Config GenerationConfig TextGenerator BeamSearch KVCache LayerKVCache FlashAttention "
                       "scaled_dot_product_attention HFLoader HFTokenizer GPT2LMHead")
    m += _missing(llm.LLaMAConfig, "llama2_7b llama2_13b llama3_8b tiny") + _missing(llm.GPT2Config, "small medium large xl tiny gpt_1_3b")
    m += _missing(llm.GenerationConfig, "greedy sampling top_k_sampling nucleus_sampling beam_search")
    m += _missing(llm.KVCache, "new update len is_empty clear") + _missing(llm.LayerKVCache, "get_mut seq_len")
    m += _missing(llm.FlashAttention, "new with_block_size forward_qkv memory_estimate")
    m += _missing(llm.HFLoader, "new from_local download_file load_config load_tensors get_tensor get_as_tensor tensor_names")
    m += _missing(llm.HFTokenizer, "from_pretrained from_directory encode decode")
    m += _missing(data.DataLoader, "new shuffle drop_last num_workers")
    m += _missing(autograd, "checkpoint checkpoint_sequential autocast no_grad Variable")
    m += _missing(jit, "trace JitCompiler compile_fn compile_graph_with_config CompileConfig Mode Backend")
    assert not m, m


def test_llama3_8b_and_gpt_1_3b_presets_match_the_benchmark_configs():
    c = llm.LLaMAConfig.llama3_8b()
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.intermediate_size,
            c.vocab_size) == (32, 4096, 32, 8, 14336, 128256) and c.rope_theta == 5e5
    g = llm.GPT2Config.gpt_1_3b()
    assert (g.n_layer, g.n_embd, g.n_head, g.n_ctx, g.vocab_size, g.intermediate_size()) == (24, 2048, 16, 2048, 50257, 8192)
