"""Built-in environment registrations."""

from ..registration import register

register("gsm8k", "skyrl_b200.gym.envs.gsm8k:GSM8kEnv", override=True)
register("gsm8k_multi_turn", "skyrl_b200.gym.envs.gsm8k:GSM8kMultiTurnEnv", override=True)
register("aime", "skyrl_b200.gym.envs.aime:AIMEEnv", override=True)
register("synthetic_bernoulli", "skyrl_b200.gym.envs.synthetic:SyntheticBernoulliEnv", override=True)
register("synthetic_gaussian", "skyrl_b200.gym.envs.synthetic:SyntheticGaussianEnv", override=True)
register("synthetic_even", "skyrl_b200.gym.envs.synthetic:SyntheticEvenEnv", override=True)
register("synthetic_multiturn", "skyrl_b200.gym.envs.synthetic:SyntheticMultiTurnEnv", override=True)
register("search", "skyrl_b200.gym.envs.tool_envs:SearchEnv", override=True)
register("searchcode", "skyrl_b200.gym.envs.tool_envs:SearchCodeEnv", override=True)
register("text2sql", "skyrl_b200.gym.envs.tool_envs:Text2SQLEnv", override=True)
register("lcb", "skyrl_b200.gym.envs.tool_envs:LiveCodeBenchEnv", override=True)
register("rlm", "skyrl_b200.gym.envs.rlm:RLMEnv", override=True)
register("llm_judge", "skyrl_b200.gym.envs.llm_judge:LLMJudgeEnv", override=True)
