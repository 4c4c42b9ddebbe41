// Command-line text generation over librllama_b200.so: rllama's `main` and
// `command_line_inference` (src/rllama_main.rs:105-347, :714-926) with the model on a B200.
//
// Same flags (src/rllama_main.rs:28-103), same start-up messages, same token loop (prefill with
// the whole prompt at position 0, then one token per call at position len-1), same colours, same
// stop rule ("</s>"), same interactive mode, same timing lines at the end. Differences:
//  * the model lives on the device: `--cuda-device` (alias `--opencl-device`) picks it,
//    `--percentage-to-gpu <p>`: layer i is resident in HBM iff i <= round(p * (n_layers - 1)), as in the reference;
//    there is no CPU path, so the other layers wait in pinned host memory and are copied to the GPU inside every forward;
//  * `--f16` alone selects f16 weights and caches (the reference's OpenCL build forces f16);
//  * `--seed` (no counterpart) seeds the sampler's draw, which the reference takes from thread_rng;
//  * `--inference-server` runs the HTTP server of inference_server.hpp (the reference: rocket).
#include <unistd.h>

#include <charconv>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <optional>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "../../include/rllama_b200.h"
#include "inference_server.hpp"

namespace {

struct Cli {
    std::string model_path, tokenizer_path, param_path;
    bool quiet = false;
    std::optional<std::string> prompt, prompt_file;
    std::optional<std::string> interactive_system_prompt, interactive_prompt_postfix, interactive_prompt_prefix;
    std::vector<std::string> interactive_stop;
    bool start_interactive = false;
    std::optional<long> max_seq_len;
    std::optional<float> temperature, top_p, repetition_penalty;
    std::optional<int> top_k;
    std::optional<long> max_threads;
    bool f16 = false;
    std::optional<long> cuda_device;
    std::optional<float> percentage_to_gpu;
    bool inference_server = false;
    std::optional<long> inference_server_port, inference_server_max_concurrent_inferences, inference_server_prompt_cache_size;
    std::optional<std::string> inference_server_host, inference_server_api_path;
    bool inference_server_exit_after_one_query = false;
    std::optional<uint64_t> seed;
};

[[noreturn]] void usage_error(const std::string& msg) {
    // clap's style: the error, a usage line, exit status 2
    std::fprintf(stderr, "error: %s\n\nUsage: rllama-b200 --model-path <MODEL_PATH> --tokenizer-path <TOKENIZER_PATH> --param-path <PARAM_PATH> [OPTIONS]\n\nFor more information, try '--help'.\n",
                 msg.c_str());
    std::exit(2);
}

void print_help() {
    std::puts(
        "Usage: rllama-b200 --model-path <MODEL_PATH> --tokenizer-path <TOKENIZER_PATH> --param-path <PARAM_PATH> [OPTIONS]\n\n"
        "Options:\n"
        "      --model-path <MODEL_PATH>\n      --tokenizer-path <TOKENIZER_PATH>\n      --param-path <PARAM_PATH>\n"
        "  -q, --quiet\n      --prompt <PROMPT>\n      --prompt-file <PROMPT_FILE>\n"
        "      --interactive-system-prompt <TEXT>\n      --interactive-stop <TEXT> (repeatable)\n"
        "      --interactive-prompt-postfix <TEXT>\n      --interactive-prompt-prefix <TEXT>\n      --start-interactive\n"
        "      --max-seq-len <N>\n      --temperature <T>\n      --top-p <P>\n      --top-k <K>\n      --repetition-penalty <R>\n"
        "      --max-threads <N>\n      --f16\n      --cuda-device <N> (alias --opencl-device)\n      --percentage-to-gpu <P>\n"
        "      --seed <N>\n      --inference-server\n      --inference-server-port <PORT>\n      --inference-server-host <HOST>\n"
        "      --inference-server-max-concurrent-inferences <N>\n      --inference-server-api-path <PATH>\n"
        "      --inference-server-prompt-cache-size <N>\n      --inference-server-exit-after-one-query\n  -h, --help");
}

template <typename T>
T parse_number(const std::string& flag, const std::string& v) {
    T out{};
    const char* b = v.data();
    const char* e = b + v.size();
    auto r = std::from_chars(b, e, out);
    if (r.ec != std::errc() || r.ptr != e) usage_error("invalid value '" + v + "' for '--" + flag + "'");
    return out;
}

Cli parse_cli(int argc, char** argv) {
    Cli c;
    bool have_model = false, have_tok = false, have_param = false;
    for (int i = 1; i < argc; i++) {
        std::string a = argv[i];
        if (a == "-h" || a == "--help") { print_help(); std::exit(0); }
        if (a == "-q") { c.quiet = true; continue; }
        if (a.rfind("--", 0) != 0) usage_error("unexpected argument '" + a + "' found");
        std::string name = a.substr(2);
        std::optional<std::string> inline_value;
        const size_t eq = name.find('=');
        if (eq != std::string::npos) { inline_value = name.substr(eq + 1); name = name.substr(0, eq); }
        auto flag = [&](bool* dst) {
            if (inline_value) usage_error("unexpected value '" + *inline_value + "' for '--" + name + "' found; no more were expected");
            *dst = true;
        };
        auto value = [&]() -> std::string {
            if (inline_value) return *inline_value;
            if (i + 1 >= argc) usage_error("a value is required for '--" + name + " <VALUE>' but none was supplied");
            return argv[++i];
        };
        if (name == "model-path") { c.model_path = value(); have_model = true; }
        else if (name == "tokenizer-path") { c.tokenizer_path = value(); have_tok = true; }
        else if (name == "param-path") { c.param_path = value(); have_param = true; }
        else if (name == "quiet") flag(&c.quiet);
        else if (name == "prompt") c.prompt = value();
        else if (name == "prompt-file") c.prompt_file = value();
        else if (name == "interactive-system-prompt") c.interactive_system_prompt = value();
        else if (name == "interactive-stop") c.interactive_stop.push_back(value());
        else if (name == "interactive-prompt-postfix") c.interactive_prompt_postfix = value();
        else if (name == "interactive-prompt-prefix") c.interactive_prompt_prefix = value();
        else if (name == "start-interactive") flag(&c.start_interactive);
        else if (name == "max-seq-len") c.max_seq_len = parse_number<long>(name, value());
        else if (name == "temperature") c.temperature = parse_number<float>(name, value());
        else if (name == "top-p") c.top_p = parse_number<float>(name, value());
        else if (name == "top-k") c.top_k = parse_number<int>(name, value());
        else if (name == "repetition-penalty") c.repetition_penalty = parse_number<float>(name, value());
        else if (name == "max-threads") c.max_threads = parse_number<long>(name, value());
        else if (name == "f16") flag(&c.f16);
        else if (name == "cuda-device" || name == "opencl-device") c.cuda_device = parse_number<long>(name, value());
        else if (name == "percentage-to-gpu") c.percentage_to_gpu = parse_number<float>(name, value());
        else if (name == "seed") c.seed = parse_number<uint64_t>(name, value());
        else if (name == "inference-server") flag(&c.inference_server);
        else if (name == "inference-server-exit-after-one-query") flag(&c.inference_server_exit_after_one_query);
        else if (name == "inference-server-port") {
            c.inference_server_port = parse_number<long>(name, value());
            if (*c.inference_server_port < 0 || *c.inference_server_port > 65535) usage_error("invalid value for '--inference-server-port': not a 16-bit port");
        }
        else if (name == "inference-server-host") c.inference_server_host = value();
        else if (name == "inference-server-max-concurrent-inferences") c.inference_server_max_concurrent_inferences = parse_number<long>(name, value());
        else if (name == "inference-server-api-path") c.inference_server_api_path = value();
        else if (name == "inference-server-prompt-cache-size") c.inference_server_prompt_cache_size = parse_number<long>(name, value());
        else usage_error("unexpected argument '--" + name + "' found");
    }
    if (!have_model || !have_tok || !have_param) {
        std::string missing;
        if (!have_model) missing += "\n  --model-path <MODEL_PATH>";
        if (!have_tok) missing += "\n  --tokenizer-path <TOKENIZER_PATH>";
        if (!have_param) missing += "\n  --param-path <PARAM_PATH>";
        usage_error("the following required arguments were not provided:" + missing);
    }
    return c;
}

// The `colored` crate's decision (its ShouldColorize::from_env): CLICOLOR_FORCE set to anything but
// "0" forces colour; else NO_COLOR set (to any value) disables it; else colour is on when CLICOLOR is
// not "0" and stdout is a terminal.
bool should_colorize() {
    auto norm = [](const char* v) -> std::optional<bool> { if (!v) return std::nullopt; return std::string(v) != "0"; };
    const auto force = norm(std::getenv("CLICOLOR_FORCE"));
    if (force && *force) return true;
    if (norm(std::getenv("NO_COLOR"))) return false;
    const auto cc = norm(std::getenv("CLICOLOR"));
    return cc.value_or(true) && isatty(STDOUT_FILENO);
}

bool g_color = false;
std::string truecolor(const std::string& s, int r, int g, int b) {
    if (!g_color || s.empty()) return s;
    char head[48];
    std::snprintf(head, sizeof head, "\x1b[38;2;%d;%d;%dm", r, g, b);
    return std::string(head) + s + "\x1b[0m";
}

// Rust's `{}` for floats: the shortest decimal that reads back, never in exponent form.
template <typename F>
std::string display_float(F v) {
    char buf[400];
    auto r = std::to_chars(buf, buf + sizeof buf, v, std::chars_format::fixed);
    return std::string(buf, r.ptr);
}

// Rust's `{:?}` for a string.
std::string debug_str(const std::string& s) {
    std::string o = "\"";
    for (char ch : s) {
        switch (ch) {
            case '\n': o += "\\n"; break;
            case '\r': o += "\\r"; break;
            case '\t': o += "\\t"; break;
            case '"': o += "\\\""; break;
            case '\\': o += "\\\\"; break;
            default: o += ch;
        }
    }
    return o + "\"";
}

std::string replace_all(std::string s, const std::string& from, const std::string& to) {
    size_t pos = 0;
    while ((pos = s.find(from, pos)) != std::string::npos) { s.replace(pos, from.size(), to); pos += to.size(); }
    return s;
}

bool ends_with(const std::string& s, const std::string& suffix) {
    return s.size() >= suffix.size() && s.compare(s.size() - suffix.size(), suffix.size(), suffix) == 0;
}

struct Failure { std::string what; };
void ok(int status) {
    if (status != RLB_OK) throw Failure{rlb_last_error()};
}

std::string read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw Failure{"No such file or directory (os error 2)"};
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

std::vector<int32_t> tokenize(rlb_tokenizer* tk, const std::string& text) {
    int32_t n = 0;
    ok(rlb_tokenizer_tokenize_to_ids(tk, text.c_str(), nullptr, 0, &n));
    std::vector<int32_t> ids((size_t)n);
    ok(rlb_tokenizer_tokenize_to_ids(tk, text.c_str(), ids.data(), n, &n));
    return ids;
}

}  // namespace

// command_line_inference (src/rllama_main.rs:714-926)
static void command_line_inference(const Cli& cli, rlb_model* model, rlb_tokenizer* tk, std::string prompt,
                                   const std::vector<std::string>& interactive_stop, const std::string& interactive_system_prompt,
                                   const std::string& interactive_prompt_prefix, const std::string& interactive_prompt_postfix,
                                   bool start_interactive, bool be_quiet, long max_seq_len, const rlb_model_params& params, int32_t vocab, long max_threads) {
    auto pln = [&](const std::string& s) { if (!be_quiet) std::printf("%s\n", s.c_str()); };

    if (start_interactive && !prompt.empty())
        throw Failure{"Cannot start interactive mode with a prompt. Use --interactive-system-prompt instead."};
    if (start_interactive) prompt = interactive_system_prompt;

    std::vector<int32_t> toks_id = tokenize(tk, prompt);
    std::string toks_str = prompt;
    size_t prev_pos = 0;
    // the loop's own defaults, not TokenSampler::new()'s (src/rllama_main.rs:753-757)
    float temperature = 1.0f, top_p = 1.0f, repetition_penalty = 1.0f;
    int32_t top_k = 20;
    if (cli.temperature) temperature = *cli.temperature;
    if (cli.top_p) top_p = *cli.top_p;
    if (cli.top_k) top_k = *cli.top_k;
    if (cli.repetition_penalty) repetition_penalty = *cli.repetition_penalty;
    rlb_sampler* sampler = nullptr;
    ok(rlb_sampler_create(&sampler));
    ok(rlb_sampler_set(sampler, temperature, top_p, top_k, repetition_penalty));
    if (cli.seed) ok(rlb_sampler_seed(sampler, *cli.seed));
    else ok(rlb_sampler_seed(sampler, (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count() ^ ((uint64_t)getpid() << 32)));

    pln("---");
    pln(" dim: " + std::to_string(params.dim));
    pln(" n_heads: " + std::to_string(params.n_heads));
    pln(" n_layers: " + std::to_string(params.n_layers));
    pln(" norm_eps: " + display_float(params.norm_eps));
    pln(" vocab_size: " + std::to_string(params.vocab_size));
    pln("---");
    pln(" maximum number of threads: " + std::to_string(max_threads));
    pln("---");
    pln("Max sequence length: " + std::to_string(max_seq_len));
    pln("Temperature: " + display_float(temperature));
    pln("Top P: " + display_float(top_p));
    pln("Top K: " + std::to_string(top_k));
    pln("Repetition penalty: " + display_float(repetition_penalty));
    if (start_interactive) {
        std::string stops = "[";
        for (size_t i = 0; i < interactive_stop.size(); i++) stops += (i ? ", " : "") + debug_str(interactive_stop[i]);
        pln("  Interactive mode stop token sequences: " + stops + "]");
        pln("---");
        pln("System prompt:");
        pln("  " + interactive_system_prompt);
        pln("---");
        pln("Interactive prompt prefix: " + interactive_prompt_prefix);
        pln("Interactive prompt postfix: " + interactive_prompt_postfix);
    }
    pln("---");
    pln(truecolor("  This is the color of the initial prompt", 128, 128, 255));
    pln(truecolor("  This is the color of the generated text", 128, 255, 128));
    pln("---");
    std::fputs(truecolor(prompt, 128, 128, 255).c_str(), stdout);
    std::fflush(stdout);

    using clock = std::chrono::steady_clock;
    long long first_token_ms = 0;
    std::vector<long long> ms_per_token;
    rlb_caches* caches = nullptr;
    ok(rlb_caches_create(model, &caches));
    std::vector<float> preds((size_t)vocab);
    bool first = true, stop_seen = false, interactive = start_interactive;
    std::vector<int32_t> user_token;
    while ((long)toks_id.size() < max_seq_len) {
        const auto now = clock::now();
        ok(rlb_forward(model, caches, toks_id.data() + prev_pos, (int32_t)(toks_id.size() - prev_pos), (int32_t)prev_pos, preds.data()));
        if (interactive) {
            std::string newinput;
            if (!std::getline(std::cin, newinput)) newinput.clear();  // read_line; the trailing newline is gone already
            newinput = interactive_prompt_prefix + newinput + interactive_prompt_postfix;
            user_token = tokenize(tk, newinput);
            user_token.erase(user_token.begin());  // the start token is in the prompt already
            interactive = false;
        }
        int32_t next = 0;
        float token_prob = 0.0f;
        if (!user_token.empty()) {
            next = user_token.front();
            user_token.erase(user_token.begin());
        } else {
            ok(rlb_sampler_sample(sampler, preds.data(), vocab, toks_id.data(), (int32_t)toks_id.size(), &next, &token_prob));
        }
        toks_id.push_back(next);

        for (size_t tok_idx = 0; prev_pos + 1 + tok_idx < toks_id.size(); tok_idx++) {
            const int32_t tok_id = toks_id[prev_pos + 1 + tok_idx];
            if (tok_id == 1) continue;
            const char* piece = nullptr;
            ok(rlb_tokenizer_id_to_str(tk, tok_id, &piece));
            const std::string tok_str = piece;
            std::string tok_print;
            if (tok_str == "</s>") stop_seen = true;
            if (tok_str == "<0x0A>") tok_print += "\n";
            else tok_print += replace_all(tok_str, "\xE2\x96\x81", " ");
            toks_str += tok_print;
            if (first && tok_idx + 2 < toks_id.size()) {
                // part of the prompt: printed already
            } else {
                float redness = token_prob * 255.0f;
                const int red = redness > 255.0f ? 255 : redness < 0.0f ? 0 : (int)redness;
                std::fputs(truecolor(tok_print, 128 + red / 2, 255 - red / 2, 128).c_str(), stdout);
            }
            for (const std::string& stop_str : interactive_stop) {
                if (!first && ends_with(toks_str, stop_str)) {
                    if (start_interactive) interactive = true;
                    break;
                }
            }
        }
        const long long ms = std::chrono::duration_cast<std::chrono::milliseconds>(clock::now() - now).count();
        if (first) first_token_ms = ms;
        else ms_per_token.push_back(ms);
        std::fflush(stdout);
        prev_pos = toks_id.size() - 1;
        first = false;
        if (stop_seen) break;
    }
    std::printf("\n");
    if (stop_seen && !be_quiet) std::printf("Stop token seen. Stopping.\n");
    if (!be_quiet) {
        std::printf("---\n");
        std::printf("Time taken to generate first token: %lldms\n", first_token_ms);
        if (!ms_per_token.empty()) {
            long long sum = 0;
            for (long long v : ms_per_token) sum += v;
            std::printf("Time taken per token (excluding first token): %lldms\n", sum / (long long)ms_per_token.size());
        } else {
            std::printf("No token generated\n");
        }
    }
    rlb_caches_free(caches);
    rlb_sampler_free(sampler);
}

// main (src/rllama_main.rs:105-347)
static void run(const Cli& cli) {
    const std::string interactive_system_prompt = cli.interactive_system_prompt.value_or(
        "A chat between a curious human and an artificial intelligence assistant. The assistant gives helpful, terse answers to the "
        "human's questions.### Human:");
    std::vector<std::string> interactive_stop = cli.interactive_stop;
    if (interactive_stop.empty()) {
        // every spelling of "### Human:" the reference looks for (src/rllama_main.rs:115-134)
        for (const char* lead : {"", " ", "\n", "\n "})
            for (const char* body : {"### Human:", "###Human:", "### Human: ", "###Human: "}) interactive_stop.push_back(std::string(lead) + body);
    }
    const std::string interactive_prompt_prefix = cli.interactive_prompt_prefix.value_or(" ");
    const std::string interactive_prompt_postfix = cli.interactive_prompt_postfix.value_or("### Assistant:");
    const long max_threads = cli.max_threads.value_or((long)std::thread::hardware_concurrency());

    bool be_quiet = !should_colorize();
    if (cli.quiet) be_quiet = true;
    g_color = !be_quiet;
    auto pln = [&](const std::string& s) { if (!be_quiet) std::printf("%s\n", s.c_str()); };

    rlb_ctx* ctx = nullptr;
    ok(rlb_ctx_create(be_quiet ? 0 : 1, (int)cli.cuda_device.value_or(0), &ctx));  // no CPU mode to fall back to
    pln("CUDA device initialized.");

    // params.json is read before the prompt so that a missing file fails first, as in the reference
    (void)read_file(cli.param_path);

    std::string prompt;
    if (cli.prompt && !cli.prompt_file) {
        pln("Using prompt: " + *cli.prompt);
        prompt = *cli.prompt;
    } else if (!cli.prompt && cli.prompt_file) {
        pln("Using prompt file: " + *cli.prompt_file);
        prompt = read_file(*cli.prompt_file);
    } else if (!(cli.start_interactive || cli.inference_server) || cli.prompt || cli.prompt_file) {
        // neither or both given; only interactive mode and the server may start without a prompt
        std::fprintf(stderr, "Please provide either a prompt or a prompt file.\n");
        throw Failure{"Please provide either a prompt or a prompt file."};
    }

    pln("Starting up. Loading tokenizer from " + cli.tokenizer_path + "...");
    rlb_tokenizer* tk = nullptr;
    ok(rlb_tokenizer_load(cli.tokenizer_path.c_str(), &tk));
    pln("Tokenizer loaded. Loading model from " + cli.model_path + "...");
    rlb_data_source* ds = nullptr;
    ok(rlb_data_source_open_inferred(cli.model_path.c_str(), &ds));  // DataSource::from_inferred_source (:239)
    rlb_model_params params;
    std::memset(&params, 0, sizeof params);
    ok(rlb_model_params_from_json(cli.param_path.c_str(), &params));
    pln("Loaded model parameters from " + cli.param_path + ".");
    const long max_seq_len = cli.max_seq_len.value_or(1024);
    params.max_seq_len = (int32_t)max_seq_len;
    params.force_f16 = cli.f16 ? 1 : 0;
    params.tp_rank = 0;
    params.tp_size = 1;
    params.has_percentage_to_gpu = 1;
    params.percentage_to_gpu = cli.percentage_to_gpu.value_or(1.0f);  // src/rllama_main.rs:160
    pln("Loading embeddings from " + cli.model_path + "...");
    pln("Loading transformer weights from " + cli.model_path + "...");
    rlb_model* model = nullptr;
    ok(rlb_model_from_llama_source(ctx, ds, &params, &model));
    rlb_data_source_free(ds);
    pln("All is loaded. Starting inference.");

    // the printed vocab_size is the file's value (-1 in Meta's params.json); the model's own comes
    // from the embedding table, and that is the length of the logits
    double vocab = 0;
    ok(rlb_model_get_stat(model, "vocab_size", &vocab));
    if (cli.inference_server) {
        // server_inference (src/rllama_main.rs:317-386)
        const long port = cli.inference_server_port.value_or(8080);
        const std::string host = cli.inference_server_host.value_or("127.0.0.1");
        const long concurrent = cli.inference_server_max_concurrent_inferences.value_or(5);
        const std::string api_path = cli.inference_server_api_path.value_or("/rllama/v1/inference");
        const long cache_size = cli.inference_server_prompt_cache_size.value_or(50);
        pln("Maximum concurrent inferences: " + std::to_string(concurrent));
        pln("Prompt cache size: " + std::to_string(cache_size));
        pln("Maximum sequence length: " + std::to_string(max_seq_len));
        pln("--- Starting HTTP server on " + host + ":" + std::to_string(port) + ", answering to requests at " + api_path + " ---");
        std::fflush(stdout);
        server::ServerState state((size_t)std::max(0L, cache_size), (size_t)std::max(1L, concurrent));
        state.model = model;
        state.tokenizer = tk;
        state.vocab = (int32_t)vocab;
        state.max_seq_len = (size_t)max_seq_len;
        state.exit_after_one_query = cli.inference_server_exit_after_one_query;
        const std::string why = server::serve(&state, host, (int)port, api_path);
        throw Failure{"Starting web server failed. (" + why + ")"};
    }
    command_line_inference(cli, model, tk, prompt, interactive_stop, interactive_system_prompt, interactive_prompt_prefix,
                           interactive_prompt_postfix, cli.start_interactive, be_quiet, max_seq_len, params, (int32_t)vocab, max_threads);
    rlb_model_free(model);
    rlb_tokenizer_free(tk);
    rlb_ctx_destroy(ctx);
}

int main(int argc, char** argv) {
    const Cli cli = parse_cli(argc, argv);
    try {
        run(cli);
    } catch (const Failure& f) {
        std::fprintf(stderr, "Error: %s\n", debug_str(f.what).c_str());  // Rust prints main's Err with {:?}
        return 1;
    }
    return 0;
}
