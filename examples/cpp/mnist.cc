// MNIST classifier on the C++ frontend: a 784-30-10 perceptron with a Sigmoid between the layers, SGD,
// batches of consecutive samples, then accuracy and mean loss over the test set — the program, the flags
// and the log lines of the reference's example/mnist/main.cc.
//
//   itb_mnist --dataset DIR [--bs 64] [--num_epoch 1] [--lr 0.01] [--device cpu|cuda] [--data_parallel N]
//
// DIR holds train-images-idx3-ubyte, train-labels-idx1-ubyte, t10k-images-idx3-ubyte and
// t10k-labels-idx1-ubyte.  --data_parallel N runs the network through the single-process DataParallel
// module over N devices (N model replicas on the CPU when --device cpu): same numbers, since the batch
// loss is the mean of equal-sized chunk losses.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <map>
#include <numeric>
#include <string>

#include "itb/itb.h"

namespace {

constexpr int kNumItersOfOutputDuration = 10;

std::map<std::string, std::string> parse(int argc, char** argv) {
  std::map<std::string, std::string> kv;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    TORCH_CHECK(a.rfind("--", 0) == 0, "unexpected argument ", a);
    a = a.substr(2);
    auto eq = a.find('=');
    if (eq != std::string::npos) kv[a.substr(0, eq)] = a.substr(eq + 1);
    else if (i + 1 < argc) kv[a] = argv[++i];
    else kv[a] = "";
  }
  return kv;
}

std::shared_ptr<itb::Module> make_network() {
  using namespace itb::nn;
  return std::make_shared<Sequential>(std::vector<std::shared_ptr<itb::Module>>{
      std::make_shared<Linear>(784, 30), std::make_shared<Sigmoid>(), std::make_shared<Linear>(30, 10)});
}

// The network proper, fed [batch, 28, 28] images.
class MNIST : public itb::Module {
 public:
  MNIST() : itb::Module("MNIST") { net_ = register_module("sequential", make_network()); }
  itb::TensorList Forward(const itb::TensorList& in) override {
    return (*net_)(itb::TensorList{in[0].reshape({in[0].size(0), 784})});
  }

 private:
  std::shared_ptr<itb::Module> net_;
};

}  // namespace

int main(int argc, char** argv) {
  auto fl = parse(argc, argv);
  auto get = [&](const std::string& k, const std::string& d) { return fl.count(k) ? fl[k] : d; };
  const std::string dir = get("dataset", "");
  TORCH_CHECK(!dir.empty(), "--dataset DIR is required");
  const int64_t bs = std::stoll(get("bs", "64")), epochs = std::stoll(get("num_epoch", "1"));
  const double lr = std::stod(get("lr", "0.01"));
  const std::string device_name = get("device", "cpu");
  TORCH_CHECK(device_name == "cpu" || device_name == "cuda", "--device must be cpu or cuda");
  const int64_t replicas = std::stoll(get("data_parallel", "1"));
  const bool cuda = device_name == "cuda";
  torch::Device device = cuda ? torch::Device(torch::kCUDA, 0) : torch::Device(torch::kCPU);

  auto train_set = std::make_shared<itb::data::MNISTDataset>(dir, /*train=*/true);
  auto test_set = std::make_shared<itb::data::MNISTDataset>(dir, /*train=*/false);
  itb::data::DataLoader train_loader(train_set, bs), test_loader(test_set, bs);

  std::shared_ptr<itb::Module> network = std::make_shared<MNIST>();
  network->To(device);
  if (replicas > 1) {
    std::vector<torch::Device> devices;
    for (int64_t i = 0; i < replicas; ++i) devices.push_back(cuda ? torch::Device(torch::kCUDA, i) : torch::Device(torch::kCPU));
    network = std::make_shared<itb::parallel::DataParallel>(network, [] { return std::make_shared<MNIST>(); }, devices);
  }
  itb::nn::CrossEntropyLoss loss_fn;
  itb::optim::SGD optimizer(network->Parameters(), lr);

  for (int64_t epoch = 0; epoch < epochs; ++epoch) {
    int64_t train_idx = 0;
    double total_loss = 0;
    const auto t0 = std::chrono::high_resolution_clock::now();
    for (auto it = train_loader.begin(); it != train_loader.end(); ++it) {
      auto [image, label] = *it;
      auto outputs = (*network)(itb::TensorList{image.to(device)});
      optimizer.ZeroGrad();
      itb::Tensor loss = loss_fn(itb::TensorList{outputs[0], label.to(device)})[0];
      const float current = loss.item<float>();
      total_loss += current;
      if (train_idx % kNumItersOfOutputDuration == 0)
        std::fprintf(stderr, "epoch: %lld, [%lld/%zu]  loss: %.6f\n", (long long)epoch, (long long)(train_idx * bs), train_set->Size(), current);
      loss.backward();
      optimizer.Step();
      ++train_idx;
    }
    const double us = std::chrono::duration<double, std::micro>(std::chrono::high_resolution_clock::now() - t0).count();
    std::fprintf(stderr, "epoch %2lld/%lld | train loss %.6f | lr %.2e | (%.2f ms | %.0f samples/s)\n", (long long)epoch,
                 (long long)(epochs - 1), total_loss / std::max<int64_t>(train_idx, 1), lr, us / 1e3, train_set->Size() / (us / 1e6));
  }

  torch::NoGradGuard no_grad;
  std::vector<float> test_losses;
  int64_t correct = 0, total = 0;
  for (auto it = test_loader.begin(); it != test_loader.end(); ++it) {
    auto [image, label] = *it;
    auto outputs = (*network)(itb::TensorList{image.to(device)});
    itb::Tensor loss = loss_fn(itb::TensorList{outputs[0], label.to(device)})[0];
    itb::Tensor predicted = outputs[0].argmax(-1).to(torch::kCPU);
    correct += predicted.eq(label.to(torch::kLong)).sum().item<int64_t>();
    total += label.size(0);
    test_losses.push_back(loss.item<float>());
  }
  const double avg = test_losses.empty() ? 0.0 : std::accumulate(test_losses.begin(), test_losses.end(), 0.0) / test_losses.size();
  std::fprintf(stderr, "Total: %lld, Correct: %lld, Accuracy: %.6f, AverageLoss: %.6f\n", (long long)total, (long long)correct,
               total ? static_cast<double>(correct) / total : 0.0, avg);
  return 0;
}
